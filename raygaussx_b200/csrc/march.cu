// Forward and backward ray march.
//
// One warp marches one ray.  The 32 lanes are the 32 samples of a slab while
// Gaussians are evaluated (every Gaussian record is then a warp-uniform shared
// memory read) and the 32 children of a hierarchy node while the hierarchy is
// searched (one coalesced load of 32 boxes per step).  Per-slab sums therefore
// live in one register per lane, compositing is a warp scan, and no per-ray hit
// list ever goes to global memory.
//
// Semantics follow the reference's OptiX programs:
//   forward   optix_raycasting/cuda_train/forward/gaussians_aabb.cu:36-340
//   backward  optix_raycasting/cuda_train/backward/gaussians_aabb.cu:113-497
//   depth     optix_raycasting/cuda_gui/gaussians_aabb.cu:189-202
// A trace over [tmin,tmax] reports Gaussian i iff the ray meets i's box within
// the interval (what OptiX traversal guarantees) and the interval test of the
// intersection program passes.  Where the reference's forward and backward
// differ, the forward's behaviour is used for both.
#include "march_common.cuh"

// This file holds the per-ray variant: every query searches the hierarchy (or,
// for validation, every Gaussian) on its own.  It is the general path -- it makes
// no assumption about neighbouring rays and needs no per-view lists -- selected by
// RGX_FLAG_PER_RAY_SEARCH / RGX_FLAG_BRUTE_FORCE and used by rgx_forward_static.

namespace rgx {

namespace {

// One ray from start to end, every query a search of the hierarchy (BRUTE: of all Gaussians).
template <bool COUNT, bool BRUTE>
__device__ __forceinline__ void march_ray_by_search(const MarchLaunch& L, int px, int py, const SceneBox& box, float eps,
                                                    float bg, WarpShared& ws, int lane, Tally& tl) {
    const int ray_id = py * L.cam.width + px;
    Ray r;
    make_ray(L.cam, px, py, r);
    float tenter, texit;
    clip_scene(box, r, tenter, texit);
    RayColor st = {1.0f, 0.f, 0.f, 0.f, 0.f};
    if (COUNT) tl.v[C_RAYS] += 1;
    float first = L.g.n > 0 ? search_closest<COUNT, BRUTE>(L, r, tenter, texit, ws, lane, tl) : INFINITY;
    if (first < INFINITY && first < texit) {                                  // :249-260
        tenter = first;
        float tbuffer = tenter;
        int slab_index = 0;
        while (tbuffer < texit && st.T > eps && slab_index < kMaxSlabs) {     // :266
            SlabPlan p = plan_slab(L.m, tbuffer, st.T, tenter, texit);
            if (COUNT) tl.v[C_SLABS] += 1;
            ++slab_index;
            if (!p.traced) { tbuffer = __fadd_rn(tbuffer, p.slab); continue; }
            const float tau = __fmul_rn((float)lane + 0.5f, p.dt);            // sample offset from tbuffer
            float s, cr, cg, cb;
            bool overflow;
            int nhit = slab_sums<COUNT, false>(L, L.m, tbuffer, tau, ray_id, slab_index, make_float3(0.f, 0.f, 0.f),
                                               ws, lane, tl, [&](auto&& leaf) {
                search_all<COUNT, BRUTE>(L, r, p.tmin, p.tmax, ws, lane, tl, leaf);
            }, s, cr, cg, cb, overflow);
            if (COUNT) { tl.v[C_HITS] += nhit; tl.v[C_OVF] += overflow ? 1 : 0; }
            if (nhit == 0) {                                                  // :297-319
                tbuffer = __fadd_rn(tbuffer, p.slab);
                float nxt = search_closest<COUNT, BRUTE>(L, r, tbuffer, texit, ws, lane, tl);
                if (!(nxt < INFINITY)) break;
                tbuffer = nxt;
                continue;
            }
            if (COUNT) tl.v[C_SLABS_HIT] += 1;
            composite_forward(p, tbuffer, tau, eps, lane, s, cr, cg, cb, L.depth != nullptr, st);
            tbuffer = __fadd_rn(tbuffer, p.slab);                             // :324
        }
    }
    if (lane == 0) {                                                           // :326-339
        write_ray(L, ray_id, st, bg);
    }
}

template <bool COUNT, bool BRUTE>
__global__ void __launch_bounds__(kWarps * 32) march_forward_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ WarpShared shared[kWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    WarpShared& ws = shared[warp];
    const int W = L.cam.width;
    const int tiles_x = (W + kTile - 1) / kTile;
    const int tile_x = blockIdx.x % tiles_x, tile_y = blockIdx.x / tiles_x;
    const int px = tile_x * kTile + warp;
    if (px >= W) return;
    const float eps = L.m.transmittance_eps;
    const float bg = L.m.white_background ? 1.0f : 0.0f;
    const SceneBox box = *L.box;
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;

    for (int k = 0; k < kTile; ++k) {
        const int py = L.m.row_begin + tile_y * kTile + k;
        if (py >= L.m.row_end) break;
        march_ray_by_search<COUNT, BRUTE>(L, px, py, box, eps, bg, ws, lane, tl);
    }
    if (COUNT) flush_tally(L, tl, lane);
}

// The rays a list march left unfinished because its lists stop at a horizon (march_lists.cu, HZ = 2): L.hz_rays
// holds their numbers, *L.hz_count how many.  They are marched again from the start by searching the hierarchy,
// which needs no lists: same hits, met in slot order instead of list order, so the colour equals that of complete
// lists to summation rounding.  Launched after every such march; returns at once when there are none.
__global__ void __launch_bounds__(kWarps * 32) march_forward_listed_rays_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ WarpShared shared[kWarps];
    const unsigned int n = *L.hz_count;
    if (n == 0u) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float eps = L.m.transmittance_eps;
    const float bg = L.m.white_background ? 1.0f : 0.0f;
    const SceneBox box = *L.box;
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;
    for (unsigned int i = blockIdx.x * kWarps + warp; i < n; i += gridDim.x * kWarps) {
        const int ray_id = L.hz_rays[i];
        march_ray_by_search<false, false>(L, ray_id % L.cam.width, ray_id / L.cam.width, box, eps, bg, shared[warp], lane, tl);
    }
}

template <bool BRUTE>
__global__ void __launch_bounds__(kWarps * 32) march_backward_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ WarpShared shared[kWarps];
    __shared__ int prim_of[kWarps][kFan];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    WarpShared& ws = shared[warp];
    const int W = L.cam.width;
    const int tiles_x = (W + kTile - 1) / kTile;
    const int tile_x = blockIdx.x % tiles_x, tile_y = blockIdx.x / tiles_x;
    const int px = tile_x * kTile + warp;
    if (px >= W) return;
    const float eps = L.m.transmittance_eps;
    const SceneBox box = *L.box;
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;

    for (int k = 0; k < kTile; ++k) {
        const int py = L.m.row_begin + tile_y * kTile + k;
        if (py >= L.m.row_end) break;
        const int ray_id = py * W + px;
        Ray r;
        make_ray(L.cam, px, py, r);
        float tenter, texit;
        clip_scene(box, r, tenter, texit);
        float first = L.g.n > 0 ? search_closest<false, BRUTE>(L, r, tenter, texit, ws, lane, tl) : INFINITY;
        if (!(first < INFINITY && first < texit)) continue;                       // backward .cu:249-254
        tenter = first;
        const float3 dl = make_float3(L.dl_drgb[3 * (size_t)ray_id], L.dl_drgb[3 * (size_t)ray_id + 1],
                                      L.dl_drgb[3 * (size_t)ray_id + 2]);
        float D = fmaf(dl.x, L.rgb_in[3 * (size_t)ray_id],
                       fmaf(dl.y, L.rgb_in[3 * (size_t)ray_id + 1], __fmul_rn(dl.z, L.rgb_in[3 * (size_t)ray_id + 2])));
        float T = 1.0f;
        float tbuffer = tenter;
        int slab_index = 0;
        while (tbuffer < texit && T > eps && slab_index < kMaxSlabs) {
            SlabPlan p = plan_slab(L.m, tbuffer, T, tenter, texit);
            ++slab_index;
            if (!p.traced) { tbuffer = __fadd_rn(tbuffer, p.slab); continue; }
            const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
            auto enumerate = [&](auto&& leaf) { search_all<false, BRUTE>(L, r, p.tmin, p.tmax, ws, lane, tl, leaf); };
            // pass 1: per-sample sigma and delta.colour sums, same arithmetic as the forward
            float s, dc, u0, u1;
            bool overflow;
            int nhit = slab_sums<false, true>(L, L.m, tbuffer, tau, ray_id, slab_index, dl, ws, lane, tl, enumerate, s,
                                              dc, u0, u1, overflow);
            if (nhit == 0) {
                tbuffer = __fadd_rn(tbuffer, p.slab);
                float nxt = search_closest<false, BRUTE>(L, r, tbuffer, texit, ws, lane, tl);
                if (!(nxt < INFINITY)) break;
                tbuffer = nxt;
                continue;
            }
            SlabBackTerms bt = slab_back_terms(s, dc, p.dt, T, D, eps, lane);
            // pass 2: same search again; gradients of every hit Gaussian
            slab_gradients(L, L.m, r, p, tbuffer, tau, dl, bt.beta, bt.gamma, ws, prim_of[warp], lane, enumerate,
                           [&](int j, const GaussGrad& g) { emit_global(L, dl, j, g, blockIdx.x); });
            // advance the ray state exactly as the forward does
            D = __fadd_rn(D, -bt.d_total);
            T = slab_exit_T(bt.tr, eps);
            tbuffer = __fadd_rn(tbuffer, p.slab);
        }
    }
}

}  // namespace

static int grid_for(const MarchLaunch& m) {
    int rows = m.m.row_end - m.m.row_begin;
    if (rows <= 0 || m.cam.width <= 0) return 0;
    return ((m.cam.width + kTile - 1) / kTile) * ((rows + kTile - 1) / kTile);
}

cudaError_t launch_march_forward_per_ray(const MarchLaunch& m, cudaStream_t s) {
    int grid = grid_for(m);
    if (grid == 0) return cudaSuccess;
    bool count = (m.m.flags & RGX_FLAG_COUNT_WORK) != 0, brute = (m.m.flags & RGX_FLAG_BRUTE_FORCE) != 0;
    if (count && brute) note_launch(), march_forward_kernel<true, true><<<grid, kWarps * 32, 0, s>>>(m);
    else if (count) note_launch(), march_forward_kernel<true, false><<<grid, kWarps * 32, 0, s>>>(m);
    else if (brute) note_launch(), march_forward_kernel<false, true><<<grid, kWarps * 32, 0, s>>>(m);
    else note_launch(), march_forward_kernel<false, false><<<grid, kWarps * 32, 0, s>>>(m);
    return cudaGetLastError();
}

cudaError_t launch_march_forward_listed_rays(const MarchLaunch& m, int ctas, cudaStream_t s) {
    if (m.g.n <= 0 || !m.hz_rays || !m.hz_count) return cudaSuccess;
    note_launch(), march_forward_listed_rays_kernel<<<ctas, kWarps * 32, 0, s>>>(m);
    return cudaGetLastError();
}

cudaError_t launch_march_backward_per_ray(const MarchLaunch& m, cudaStream_t s) {
    int grid = grid_for(m);
    if (grid == 0) return cudaSuccess;
    bool brute = (m.m.flags & RGX_FLAG_BRUTE_FORCE) != 0;
    if (brute) note_launch(), march_backward_kernel<true><<<grid, kWarps * 32, 0, s>>>(m);
    else note_launch(), march_backward_kernel<false><<<grid, kWarps * 32, 0, s>>>(m);
    return cudaGetLastError();
}

}  // namespace rgx
