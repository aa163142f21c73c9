// Tiled forward and backward ray march: the default path.
//
// A CTA owns an 8x8 pixel tile (RGX_TILE_X x RGX_TILE_Y).  All rays of a tile start at the eye and stay
// inside a thin pyramid, so instead of searching the hierarchy once per ray and
// per slab, the CTA searches it once per *depth window*: all eight warps sweep
// the hierarchy level by level with the tile's pyramid, cut to the window's
// depth range, and leave the Gaussians they find in a shared candidate list.
// Every ray of the tile then marches the slabs that lie inside the window against
// that list -- one warp per ray, lanes = samples, exactly as in the per-ray
// kernels -- and the CTA moves on to the next window.  The search cost is thus
// shared by 64 rays and several slabs.
//
// The candidate list is a superset of what any ray of the tile can hit inside the
// window; the per-ray test that decides a hit is the same as in the per-ray and
// exhaustive variants and candidates are kept in ascending sorted order, so all
// three variants produce identical hit sequences.  If a window's candidates do not
// fit (very deep overlap), the tile advances by per-ray hierarchy searches instead.
//
// Reference semantics: cuda_train/forward/gaussians_aabb.cu:205-340 and
// cuda_train/backward/gaussians_aabb.cu:209-497 (see march_common.cuh).
#include "march_common.cuh"

#ifndef RGX_TILE_X
#define RGX_TILE_X 8
#endif
#ifndef RGX_TILE_Y
#define RGX_TILE_Y 8
#endif

namespace rgx {

namespace {

constexpr int kTileX = RGX_TILE_X, kTileY = RGX_TILE_Y;   // pixels per CTA tile
constexpr int kRays = kTileX * kTileY;
constexpr int kCand = 2048;       // candidate Gaussians per window
constexpr int kFront = 512;       // hierarchy nodes per level per window
constexpr int kMaxWindows = 1 << 20;
constexpr int kThreads = kWarps * 32;
enum { M_DONE = 0, M_SEEK_FIRST = 1, M_SEEK = 2, M_MARCH = 3 };

struct TileShared {
    // per-ray state, saved between windows
    float t[kRays];          // SEEK*: start of the closest-hit query; MARCH: tbuffer
    float T[kRays], Cr[kRays], Cg[kRays], Cb[kRays], depth[kRays], D[kRays];
    float tenter[kRays], texit[kRays];
    int mode[kRays];
    int slab_index[kRays];
    // tile pyramid: inward plane normals through the eye, and n.o
    float pn[4][3];
    float pno[4];
    // window
    float w_lo, w_hi;
    unsigned lo_bits, slab_bits, u_bits, first_bits;
    int n_active, n_march, n_cand, n_front, overflow, next_ray, mult;
    int cand[kCand];
    float cand_lo[kCand], cand_hi[kCand];   // distance range of each candidate's box from the eye
    int pend[kWarps][2 * kFan];
    int frontier[2][kFront];
    unsigned masks[kFront];
    int offs[kFront];
    int warp_tot[kWarps];
    int prim_of[kWarps][kFan];
    WarpShared ws[kWarps];
};

// Conservative test of a box against the tile pyramid and a depth range measured
// from the eye (ray parameters are distances because directions are unit vectors).
__device__ __forceinline__ bool pyramid_box(const TileShared& sh, float3 o, float2 bx, float2 by, float2 bz, float w_lo,
                                            float bound, float& dmin, float& dmax) {
    if (!(bx.x <= bx.y)) return false;             // inverted box: padding or a culled Gaussian
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float nx = sh.pn[i][0], ny = sh.pn[i][1], nz = sh.pn[i][2];
        float ax = fmaxf(nx * bx.x, nx * bx.y), ay = fmaxf(ny * by.x, ny * by.y), az = fmaxf(nz * bz.x, nz * bz.y);
        float reach = ax + ay + az - sh.pno[i];
        float mag = fabsf(ax) + fabsf(ay) + fabsf(az) + fabsf(sh.pno[i]);
        if (reach < -1e-5f * mag) return false;
    }
    float nearx = fmaxf(fmaxf(bx.x - o.x, o.x - bx.y), 0.f), neary = fmaxf(fmaxf(by.x - o.y, o.y - by.y), 0.f),
          nearz = fmaxf(fmaxf(bz.x - o.z, o.z - bz.y), 0.f);
    float farx = fmaxf(fabsf(bx.x - o.x), fabsf(bx.y - o.x)), fary = fmaxf(fabsf(by.x - o.y), fabsf(by.y - o.y)),
          farz = fmaxf(fabsf(bz.x - o.z), fabsf(bz.y - o.z));
    dmin = sqrtf(nearx * nearx + neary * neary + nearz * nearz) * (1.0f - 1e-5f) - 1e-6f;
    dmin = fmaxf(dmin, 0.f);
    dmax = sqrtf(farx * farx + fary * fary + farz * farz) * (1.0f + 1e-5f) + 1e-6f;
    return dmax >= w_lo && dmin <= bound;
}

__device__ __forceinline__ void tile_pyramid(const rgx_camera& c, int px0, int px1, int py0, int py1, TileShared& sh) {
    // pixel-centre extremes of the tile in the image-plane coordinates of make_ray, widened a little
    float a0 = 2.0f * (((float)px0 + 0.5f) / (float)c.width - c.pp[0]) * c.tan_half_fov[0];
    float a1 = 2.0f * (((float)px1 + 0.5f) / (float)c.width - c.pp[0]) * c.tan_half_fov[0];
    float b0 = 2.0f * (((float)py0 + 0.5f) / (float)c.height - c.pp[1]) * c.tan_half_fov[1];
    float b1 = 2.0f * (((float)py1 + 0.5f) / (float)c.height - c.pp[1]) * c.tan_half_fov[1];
    float lo_a = fminf(a0, a1), hi_a = fmaxf(a0, a1), lo_b = fminf(b0, b1), hi_b = fmaxf(b0, b1);
    lo_a -= 1e-5f * (1.0f + fabsf(lo_a)); hi_a += 1e-5f * (1.0f + fabsf(hi_a));
    lo_b -= 1e-5f * (1.0f + fabsf(lo_b)); hi_b += 1e-5f * (1.0f + fabsf(hi_b));
    for (int k = 0; k < 3; ++k) {
        sh.pn[0][k] = c.u[k] - lo_a * c.w[k];     // x_cam >= lo_a * z_cam
        sh.pn[1][k] = -c.u[k] + hi_a * c.w[k];    // x_cam <= hi_a * z_cam
        sh.pn[2][k] = c.v[k] - lo_b * c.w[k];
        sh.pn[3][k] = -c.v[k] + hi_b * c.w[k];
    }
    for (int i = 0; i < 4; ++i) sh.pno[i] = sh.pn[i][0] * c.eye[0] + sh.pn[i][1] * c.eye[1] + sh.pn[i][2] * c.eye[2];
}

// Block-wide exclusive scan of popc(masks[0..n)) into offs; returns the total.  n <= kFront.
__device__ __forceinline__ int scan_masks(TileShared& sh, int n) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int per = kFront / kThreads;   // 4
    int base = tid * per, local[per], sum = 0;
#pragma unroll
    for (int i = 0; i < per; ++i) {
        int k = base + i;
        local[i] = k < n ? __popc(sh.masks[k]) : 0;
        sum += local[i];
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) sh.warp_tot[warp] = incl;
    __syncthreads();
    int woff = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        int v = sh.warp_tot[w];
        if (w < warp) woff += v;
        total += v;
    }
    int run = woff + incl - sum;
#pragma unroll
    for (int i = 0; i < per; ++i) {
        int k = base + i;
        if (k < n) sh.offs[k] = run;
        run += local[i];
    }
    __syncthreads();
    return total;
}

// Smallest distance from the eye at which the tile pyramid meets a Gaussian box that
// reaches depth w_lo or beyond; +inf if there is none.  Nearest-first descent by one
// warp, pruned by the best distance found so far.
template <bool COUNT>
__device__ float beam_first(const MarchLaunch& L, const TileShared& sh, float3 o, float w_lo, WarpShared& ws, int lane,
                            Tally& tl) {
    const Hierarchy& h = L.h;
    const int top = h.num_levels - 1;
    float best = INFINITY;
    int sp = 0;
    auto push = [&](bool pass, float dmin, int level, int c) {
        unsigned key = pass ? __float_as_uint(dmin) : 0xffffffffu;
        unsigned mn = __reduce_min_sync(kFull, key);
        unsigned near_mask = __ballot_sync(kFull, pass && key == mn);
        int near_lane = __ffs(near_mask) - 1;
        bool other = pass && lane != near_lane;
        unsigned m = __ballot_sync(kFull, other);
        int n = __popc(m), total = n + (near_lane >= 0 ? 1 : 0);
        if (sp + total > kStack) { tl.v[C_STACK_OVF] += 1; return; }
        if (other) {
            int s = sp + __popc(m & ((1u << lane) - 1u));
            ws.stack[s] = ((uint32_t)level << 26) | (uint32_t)c;
            ws.stack_t[s] = dmin;
        }
        if (lane == near_lane) {
            ws.stack[sp + n] = ((uint32_t)level << 26) | (uint32_t)c;
            ws.stack_t[sp + n] = dmin;
        }
        sp += total;
        __syncwarp();
    };
    {
        bool pass = false;
        float dmin = 0.f, dmax = 0.f;
        if (lane < h.count[top]) {
            int idx = h.offset[top] + lane;
            pass = pyramid_box(sh, o, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), w_lo, INFINITY, dmin, dmax);
        }
        if (COUNT) tl.v[C_NODE_TESTS] += h.count[top];
        push(pass, dmin, top, lane);
    }
    while (sp > 0) {
        --sp;
        uint32_t e = ws.stack[sp];
        float te = ws.stack_t[sp];
        if (te >= best) continue;
        int level = (int)(e >> 26) - 1;
        int c = (int)(e & 0x3ffffffu) * kFan + lane;
        bool pass = false;
        float dmin = 0.f, dmax = 0.f;
        if (c < h.count[level]) {
            int idx = h.offset[level] + c;
            pass = pyramid_box(sh, o, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), w_lo, best, dmin, dmax);
        }
        if (level == 0) {
            if (COUNT) tl.v[C_PRIM_TESTS] += 32;
            best = fminf(best, warp_min_f(pass ? dmin : INFINITY));
            if (best <= w_lo) break;
        } else {
            if (COUNT) tl.v[C_NODE_TESTS] += 32;
            push(pass, dmin, level, c);
        }
    }
    return best;
}

// Level-by-level sweep of the hierarchy with the tile pyramid over the depth range
// [w_lo, bound].  Leaves the candidates in sh.cand (ascending) with their depth
// ranges, their number in sh.n_cand, and sh.overflow = 1 if a level did not fit.
// Must be called by all threads of the CTA.
template <bool COUNT>
__device__ void gather_window(const MarchLaunch& L, TileShared& sh, float3 o, float w_lo, float bound, Tally& tl) {
    const Hierarchy& h = L.h;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int top = h.num_levels - 1;
    if (tid == 0) {
        sh.overflow = 0;
        sh.n_cand = 0;
    }
    if (warp == 0) {
        bool pass = false;
        float dmin = 0.f, dmax = 0.f;
        if (lane < h.count[top]) {
            int idx = h.offset[top] + lane;
            pass = pyramid_box(sh, o, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), w_lo, bound, dmin, dmax);
        }
        unsigned m = __ballot_sync(kFull, pass);
        if (pass) sh.frontier[0][__popc(m & ((1u << lane) - 1u))] = lane;
        if (lane == 0) sh.n_front = __popc(m);
        if (COUNT) tl.v[C_NODE_TESTS] += h.count[top];
    }
    __syncthreads();
    int cur = 0;
    for (int level = top; level >= 1; --level) {
        const int child_level = level - 1;
        const int nfront = sh.n_front;
        // pass 1: which children pass
        for (int k = warp; k < nfront; k += kWarps) {
            int c = sh.frontier[cur][k] * kFan + lane;
            bool pass = false;
            float dmin = 0.f, dmax = 0.f;
            if (c < h.count[child_level]) {
                int idx = h.offset[child_level] + c;
                pass = pyramid_box(sh, o, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), w_lo, bound, dmin, dmax);
            }
            unsigned m = __ballot_sync(kFull, pass);
            if (lane == 0) sh.masks[k] = m;
            if (COUNT) { if (child_level == 0) tl.v[C_PRIM_TESTS] += 32; else tl.v[C_NODE_TESTS] += 32; }
        }
        __syncthreads();
        int total = scan_masks(sh, nfront);
        const int cap = child_level == 0 ? kCand : kFront;
        if (total > cap) {
            if (tid == 0) sh.overflow = 1;
            __syncthreads();
            return;
        }
        // pass 2: write the passing children in ascending order
        int* out = child_level == 0 ? sh.cand : sh.frontier[cur ^ 1];
        for (int k = warp; k < nfront; k += kWarps) {
            unsigned m = sh.masks[k];
            if ((m >> lane) & 1u) {
                int c = sh.frontier[cur][k] * kFan + lane;
                int slot = sh.offs[k] + __popc(m & ((1u << lane) - 1u));
                out[slot] = c;
                if (child_level == 0) {
                    float dmin, dmax;
                    pyramid_box(sh, o, __ldg(&h.bx[c]), __ldg(&h.by[c]), __ldg(&h.bz[c]), w_lo, bound, dmin, dmax);
                    sh.cand_lo[slot] = dmin;
                    sh.cand_hi[slot] = dmax;
                }
            }
        }
        if (tid == 0) {
            if (child_level == 0) sh.n_cand = total; else sh.n_front = total;
        }
        __syncthreads();
        cur ^= 1;
    }
}

// A window of the tile: decides its depth range and fills the candidate list.
// With rays in mid-march the window starts at the smallest pending depth; when every
// active ray is looking for its next hit it starts at the first occupied depth.
// Returns false when nothing is left at or beyond w_lo (every active ray misses).
template <bool COUNT>
__device__ bool open_window(const MarchLaunch& L, TileShared& sh, float3 o, Tally& tl) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float start = __uint_as_float(sh.lo_bits);
    if (sh.n_march == 0) {
        if (warp == 0) {
            float f = beam_first<COUNT>(L, sh, o, start, sh.ws[0], lane, tl);
            if (lane == 0) sh.first_bits = __float_as_uint(f);
        }
        __syncthreads();
        float f = __uint_as_float(sh.first_bits);
        if (!(f < INFINITY)) return false;
        start = fmaxf(start, f);
    }
    const float w_hi = start + (float)sh.mult * __uint_as_float(sh.slab_bits);
    __syncthreads();
    if (tid == 0) { sh.w_lo = start; sh.w_hi = w_hi; }
    gather_window<COUNT>(L, sh, o, start, w_hi, tl);
    return true;
}

// Set-up shared by both passes: ray generation, scene clip, initial state.
__device__ __forceinline__ bool tile_rays_begin(const MarchLaunch& L, TileShared& sh, int tile_x, int tile_y, int& px0,
                                                int& py0) {
    const int tid = threadIdx.x;
    const int W = L.cam.width;
    px0 = tile_x * kTileX;
    py0 = L.m.row_begin + tile_y * kTileY;
    const int px1 = min(px0 + kTileX, W) - 1, py1 = min(py0 + kTileY, L.m.row_end) - 1;
    if (tid == 0) {
        tile_pyramid(L.cam, px0, px1, py0, py1, sh);
        sh.mult = 2;
    }
    for (int ray = tid; ray < kRays; ray += kThreads) {
        const int px = px0 + ray % kTileX, py = py0 + ray / kTileX;
        int mode = M_DONE;
        float tenter = 0.f, texit = 0.f;
        if (px < W && py < L.m.row_end) {
            Ray r;
            make_ray(L.cam, px, py, r);
            const SceneBox box = *L.box;
            clip_scene(box, r, tenter, texit);
            mode = (L.g.n > 0 && tenter <= texit) ? M_SEEK_FIRST : M_DONE;   // an empty first query is a miss
        }
        sh.mode[ray] = mode;
        sh.t[ray] = tenter;
        sh.tenter[ray] = tenter;
        sh.texit[ray] = texit;
        sh.T[ray] = 1.0f;
        sh.Cr[ray] = sh.Cg[ray] = sh.Cb[ray] = sh.depth[ray] = sh.D[ray] = 0.f;
        sh.slab_index[ray] = 0;
    }
    __syncthreads();
    return true;
}

// Start of a window: smallest pending depth and longest pending slab over the
// rays still active.  Returns false when the tile is finished.
__device__ __forceinline__ bool window_begin(const MarchLaunch& L, TileShared& sh) {
    const int tid = threadIdx.x;
    if (tid == 0) {
        sh.lo_bits = 0x7f800000u;
        sh.slab_bits = 0u;
        sh.n_active = 0;
        sh.n_march = 0;
        sh.next_ray = 0;
    }
    __syncthreads();
    for (int ray = tid; ray < kRays; ray += kThreads) {
        if (sh.mode[ray] == M_DONE) continue;
        float t = sh.t[ray];
        float T = sh.mode[ray] == M_MARCH ? sh.T[ray] : 1.0f;
        SlabPlan p = plan_slab(L.m, t, T, t, INFINITY);
        atomicMin(&sh.lo_bits, __float_as_uint(fmaxf(t, 0.f)));
        atomicMax(&sh.slab_bits, __float_as_uint(p.slab));
        atomicAdd(&sh.n_active, 1);
        if (sh.mode[ray] == M_MARCH) atomicAdd(&sh.n_march, 1);
    }
    __syncthreads();
    return sh.n_active > 0;
}

// ---------------------------------------------------------------- forward
template <bool COUNT>
__global__ void __launch_bounds__(kThreads) march_forward_tiled_kernel(const __grid_constant__ MarchLaunch L) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TileShared& sh = *reinterpret_cast<TileShared*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    WarpShared& ws = sh.ws[warp];
    const int W = L.cam.width;
    const int tiles_x = (W + kTileX - 1) / kTileX;
    const int tile_x = blockIdx.x % tiles_x, tile_y = blockIdx.x / tiles_x;
    const float eps = L.m.transmittance_eps;
    const float bg = L.m.white_background ? 1.0f : 0.0f;
    const float3 eye = make_float3(L.cam.eye[0], L.cam.eye[1], L.cam.eye[2]);
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;
    int px0, py0;
    const long long c_k0 = COUNT ? clock64() : 0;
    tile_rays_begin(L, sh, tile_x, tile_y, px0, py0);

    for (int win = 0; win < kMaxWindows; ++win) {
        if (!window_begin(L, sh)) break;
        const long long c_w0 = COUNT ? clock64() : 0;
        const bool something_left = open_window<COUNT>(L, sh, eye, tl);
        const bool overflow = something_left && sh.overflow != 0;
        if (COUNT) tl.v[C_CYC_WINDOW] += clock64() - c_w0;
        if (COUNT && warp == 0) {       // tallies are per warp: every lane keeps the same value
            tl.v[C_WINDOWS] += 1;
            tl.v[C_RESERVED] += sh.n_active;
            if (overflow) tl.v[sh.mult > 1 ? C_RETRIES : C_FALLBACKS] += 1;
            else if (something_left) tl.v[C_CANDS] += sh.n_cand;
        }
        if (overflow && sh.mult > 1) {              // too many candidates: try a shallower window
            __syncthreads();
            if (tid == 0) sh.mult = sh.mult / 2;
            __syncthreads();
            continue;
        }
        const int n_cand = (overflow || !something_left) ? 0 : sh.n_cand;
        const float w_hi = sh.w_hi;
        const bool exhausted = !something_left;            // nothing at or beyond the pending depths inside the pyramid
        const CandList cl = {sh.cand, sh.cand_lo, sh.cand_hi, n_cand, sh.pend[warp]};
        // every warp takes rays until none is left
        while (true) {
            int ray = 0;
            if (lane == 0) ray = atomicAdd(&sh.next_ray, 1);
            ray = __shfl_sync(kFull, ray, 0);
            if (ray >= kRays) break;
            int mode = sh.mode[ray];
            if (mode == M_DONE) continue;
            const int px = px0 + ray % kTileX, py = py0 + ray / kTileX;
            const int ray_id = py * W + px;
            Ray r;
            make_ray(L.cam, px, py, r);
            float t = sh.t[ray], tenter = sh.tenter[ray];
            const float texit = sh.texit[ray];
            RayColor st = {sh.T[ray], sh.Cr[ray], sh.Cg[ray], sh.Cb[ray], sh.depth[ray]};
            int slab_index = sh.slab_index[ray];
            if (exhausted) {
                mode = M_DONE;                       // a miss ends the march (:249-256, :314-316)
            } else {
                int steps = 0;                       // per-ray searches are limited to one step per window
                while (mode != M_DONE) {
                    if (mode == M_SEEK_FIRST || mode == M_SEEK) {
                        float found;
                        if (overflow) {
                            if (steps++ > 0) break;
                            found = search_closest<COUNT, false>(L, r, t, texit, ws, lane, tl);
                            if (!(found < INFINITY)) { mode = M_DONE; break; }
                        } else {
                            const long long c_s0 = COUNT ? clock64() : 0;
                            found = closest_in_list<COUNT>(L, r, t, texit, cl, lane, tl);
                            if (!(found <= w_hi)) {
                                // The list is only complete up to w_hi and this ray's next hit lies beyond it:
                                // look it up with a search of its own instead of trailing the windows through
                                // what may be a long stretch of empty space.
                                found = search_closest<COUNT, false>(L, r, t, texit, ws, lane, tl);
                                if (!(found < INFINITY)) { mode = M_DONE; break; }
                            }
                            if (COUNT) tl.v[C_CYC_SEEK] += clock64() - c_s0;
                        }
                        if (COUNT) tl.v[C_CLOSEST] += 1;
                        if (mode == M_SEEK_FIRST) {
                            if (!(found < texit)) { mode = M_DONE; break; }           // :260, :333-339
                            tenter = found;
                        }
                        t = found;
                        mode = M_MARCH;
                    } else {
                        if (!(t < texit && st.T > eps && slab_index < kMaxSlabs)) { mode = M_DONE; break; }   // :266
                        SlabPlan p = plan_slab(L.m, t, st.T, tenter, texit);
                        if (!p.traced) {
                            t = __fadd_rn(t, p.slab);
                            ++slab_index;
                            if (COUNT) tl.v[C_SLABS] += 1;
                            continue;
                        }
                        if (overflow) { if (steps++ > 0) break; }
                        else if (!(p.tmax <= w_hi)) break;                            // wait for the next window
                        ++slab_index;
                        if (COUNT) tl.v[C_SLABS] += 1;
                        const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
                        float s, cr, cg, cb;
                        bool ovf;
                        const long long c_q0 = COUNT ? clock64() : 0;
                        const unsigned long long ev0 = tl.v[C_CYC_EVAL];
                        int nhit = slab_sums<COUNT, false>(L, L.m, t, tau, ray_id, slab_index, make_float3(0.f, 0.f, 0.f),
                                                           ws, lane, tl, [&](auto&& leaf) {
                            if (overflow) search_all<COUNT, false>(L, r, p.tmin, p.tmax, ws, lane, tl, leaf);
                            else search_list<COUNT>(L, r, p.tmin, p.tmax, cl, lane, tl, leaf);
                        }, s, cr, cg, cb, ovf);
                        const long long c_q1 = COUNT ? clock64() : 0;
                        if (COUNT) tl.v[C_CYC_SEARCH] += (c_q1 - c_q0) - (tl.v[C_CYC_EVAL] - ev0);
                        if (COUNT) { tl.v[C_HITS] += nhit; tl.v[C_OVF] += ovf ? 1 : 0; }
                        if (nhit == 0) {                                              // :297-319
                            t = __fadd_rn(t, p.slab);
                            mode = M_SEEK;
                            continue;
                        }
                        if (COUNT) tl.v[C_SLABS_HIT] += 1;
                        composite_forward(p, t, tau, eps, lane, s, cr, cg, cb, L.depth != nullptr, st);
                        t = __fadd_rn(t, p.slab);                                     // :324
                        if (COUNT) tl.v[C_CYC_COMP] += clock64() - c_q1;
                    }
                }
            }
            if (lane == 0) {
                sh.mode[ray] = mode; sh.t[ray] = t; sh.tenter[ray] = tenter; sh.slab_index[ray] = slab_index;
                sh.T[ray] = st.T; sh.Cr[ray] = st.Cr; sh.Cg[ray] = st.Cg; sh.Cb[ray] = st.Cb; sh.depth[ray] = st.depth;
            }
        }
        const long long c_b0 = COUNT ? clock64() : 0;
        __syncthreads();
        if (COUNT) tl.v[C_CYC_WAIT] += clock64() - c_b0;
        if (tid == 0) {        // adapt the window depth to the candidate density
            // deeper windows pay off when few rays are left to scan the list
            const int na = sh.n_active;
            const int high = na >= 32 ? kCand / 2 : (na >= 8 ? (3 * kCand) / 4 : kCand);
            if (overflow) sh.mult = 1;
            else if (n_cand < high / 3 && sh.mult < 256) sh.mult *= 2;
            else if (n_cand > high && sh.mult > 1) sh.mult /= 2;
        }
        __syncthreads();
    }
    for (int ray = tid; ray < kRays; ray += kThreads) {                                // :326-339
        const int px = px0 + ray % kTileX, py = py0 + ray / kTileX;
        if (px < W && py < L.m.row_end) {
            const size_t ray_id = (size_t)py * W + px;
            const float T = sh.T[ray];
            L.rgb[3 * ray_id] = fmaf(T, bg, sh.Cr[ray]);
            L.rgb[3 * ray_id + 1] = fmaf(T, bg, sh.Cg[ray]);
            L.rgb[3 * ray_id + 2] = fmaf(T, bg, sh.Cb[ray]);
            if (L.alpha) L.alpha[ray_id] = 1.0f - T;
            if (L.depth) L.depth[ray_id] = sh.depth[ray];
            if (COUNT) atomicAdd(&L.counters->v[C_RAYS], 1ull);
        }
    }
    if (COUNT) {
        tl.v[C_CYC_TOTAL] += clock64() - c_k0;
        flush_tally(L, tl, lane);
    }
}

// ---------------------------------------------------------------- backward
__global__ void __launch_bounds__(kThreads) march_backward_tiled_kernel(const __grid_constant__ MarchLaunch L) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TileShared& sh = *reinterpret_cast<TileShared*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    WarpShared& ws = sh.ws[warp];
    const int W = L.cam.width;
    const int tiles_x = (W + kTileX - 1) / kTileX;
    const int tile_x = blockIdx.x % tiles_x, tile_y = blockIdx.x / tiles_x;
    const float eps = L.m.transmittance_eps;
    const float3 eye = make_float3(L.cam.eye[0], L.cam.eye[1], L.cam.eye[2]);
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;
    int px0, py0;
    tile_rays_begin(L, sh, tile_x, tile_y, px0, py0);
    for (int ray = tid; ray < kRays; ray += kThreads) {
        if (sh.mode[ray] == M_DONE) continue;
        const int px = px0 + ray % kTileX, py = py0 + ray / kTileX;
        const size_t ray_id = (size_t)py * W + px;
        sh.D[ray] = fmaf(L.dl_drgb[3 * ray_id], L.rgb_in[3 * ray_id],
                         fmaf(L.dl_drgb[3 * ray_id + 1], L.rgb_in[3 * ray_id + 1],
                              __fmul_rn(L.dl_drgb[3 * ray_id + 2], L.rgb_in[3 * ray_id + 2])));
    }
    __syncthreads();

    for (int win = 0; win < kMaxWindows; ++win) {
        if (!window_begin(L, sh)) break;
        const bool something_left = open_window<false>(L, sh, eye, tl);
        const bool overflow = something_left && sh.overflow != 0;
        if (overflow && sh.mult > 1) {
            __syncthreads();
            if (tid == 0) sh.mult = sh.mult / 2;
            __syncthreads();
            continue;
        }
        const int n_cand = (overflow || !something_left) ? 0 : sh.n_cand;
        const float w_hi = sh.w_hi;
        const bool exhausted = !something_left;
        const CandList cl = {sh.cand, sh.cand_lo, sh.cand_hi, n_cand, sh.pend[warp]};
        while (true) {
            int ray = 0;
            if (lane == 0) ray = atomicAdd(&sh.next_ray, 1);
            ray = __shfl_sync(kFull, ray, 0);
            if (ray >= kRays) break;
            int mode = sh.mode[ray];
            if (mode == M_DONE) continue;
            const int px = px0 + ray % kTileX, py = py0 + ray / kTileX;
            const int ray_id = py * W + px;
            Ray r;
            make_ray(L.cam, px, py, r);
            float t = sh.t[ray], tenter = sh.tenter[ray], T = sh.T[ray], D = sh.D[ray];
            const float texit = sh.texit[ray];
            int slab_index = sh.slab_index[ray];
            const float3 dl = make_float3(L.dl_drgb[3 * (size_t)ray_id], L.dl_drgb[3 * (size_t)ray_id + 1],
                                          L.dl_drgb[3 * (size_t)ray_id + 2]);
            if (exhausted) {
                mode = M_DONE;
            } else {
                int steps = 0;
                while (mode != M_DONE) {
                    if (mode == M_SEEK_FIRST || mode == M_SEEK) {
                        float found;
                        if (overflow) {
                            if (steps++ > 0) break;
                            found = search_closest<false, false>(L, r, t, texit, ws, lane, tl);
                            if (!(found < INFINITY)) { mode = M_DONE; break; }
                        } else {
                            found = closest_in_list<false>(L, r, t, texit, cl, lane, tl);
                            if (!(found <= w_hi)) {
                                found = search_closest<false, false>(L, r, t, texit, ws, lane, tl);
                                if (!(found < INFINITY)) { mode = M_DONE; break; }
                            }
                        }
                        if (mode == M_SEEK_FIRST) {
                            if (!(found < texit)) { mode = M_DONE; break; }
                            tenter = found;
                        }
                        t = found;
                        mode = M_MARCH;
                    } else {
                        if (!(t < texit && T > eps && slab_index < kMaxSlabs)) { mode = M_DONE; break; }
                        SlabPlan p = plan_slab(L.m, t, T, tenter, texit);
                        if (!p.traced) { t = __fadd_rn(t, p.slab); ++slab_index; continue; }
                        if (overflow) { if (steps++ > 0) break; }
                        else if (!(p.tmax <= w_hi)) break;
                        ++slab_index;
                        const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
                        auto enumerate = [&](auto&& leaf) {
                            if (overflow) search_all<false, false>(L, r, p.tmin, p.tmax, ws, lane, tl, leaf);
                            else search_list<false>(L, r, p.tmin, p.tmax, cl, lane, tl, leaf);
                        };
                        float s, dc, u0, u1;
                        bool ovf;
                        int nhit = slab_sums<false, true>(L, L.m, t, tau, ray_id, slab_index, dl, ws, lane, tl, enumerate,
                                                          s, dc, u0, u1, ovf);
                        if (nhit == 0) {
                            t = __fadd_rn(t, p.slab);
                            mode = M_SEEK;
                            continue;
                        }
                        SlabBackTerms bt = slab_back_terms(s, dc, p.dt, T, D, eps, lane);
                        slab_gradients(L, L.m, r, p, t, tau, dl, bt.beta, bt.gamma, ws, sh.prim_of[warp], lane, enumerate,
                                       [&](int j, const GaussGrad& g) { emit_global(L, dl, j, g); });
                        D = __fadd_rn(D, -bt.d_total);
                        T = slab_exit_T(bt.tr, eps);
                        t = __fadd_rn(t, p.slab);
                    }
                }
            }
            if (lane == 0) {
                sh.mode[ray] = mode; sh.t[ray] = t; sh.tenter[ray] = tenter; sh.slab_index[ray] = slab_index;
                sh.T[ray] = T; sh.D[ray] = D;
            }
        }
        __syncthreads();
        if (tid == 0) {
            // deeper windows pay off when few rays are left to scan the list
            const int na = sh.n_active;
            const int high = na >= 32 ? kCand / 2 : (na >= 8 ? (3 * kCand) / 4 : kCand);
            if (overflow) sh.mult = 1;
            else if (n_cand < high / 3 && sh.mult < 256) sh.mult *= 2;
            else if (n_cand > high && sh.mult > 1) sh.mult /= 2;
        }
        __syncthreads();
    }
}

int tiled_grid(const MarchLaunch& m) {
    int rows = m.m.row_end - m.m.row_begin;
    if (rows <= 0 || m.cam.width <= 0) return 0;
    return ((m.cam.width + kTileX - 1) / kTileX) * ((rows + kTileY - 1) / kTileY);
}

}  // namespace

cudaError_t launch_march_forward_per_ray(const MarchLaunch& m, cudaStream_t s);
cudaError_t launch_march_backward_per_ray(const MarchLaunch& m, cudaStream_t s);

cudaError_t launch_march_forward(const MarchLaunch& m, cudaStream_t s) {
    if (m.m.flags & (RGX_FLAG_BRUTE_FORCE | RGX_FLAG_PER_RAY_SEARCH)) return launch_march_forward_per_ray(m, s);
    int grid = tiled_grid(m);
    if (grid == 0) return cudaSuccess;
    const size_t smem = sizeof(TileShared);
    cudaError_t e;
    if (m.m.flags & RGX_FLAG_COUNT_WORK) {
        e = cudaFuncSetAttribute(march_forward_tiled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        march_forward_tiled_kernel<true><<<grid, kThreads, smem, s>>>(m);
    } else {
        e = cudaFuncSetAttribute(march_forward_tiled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        march_forward_tiled_kernel<false><<<grid, kThreads, smem, s>>>(m);
    }
    return cudaGetLastError();
}

cudaError_t launch_march_backward(const MarchLaunch& m, cudaStream_t s) {
    if (m.m.flags & (RGX_FLAG_BRUTE_FORCE | RGX_FLAG_PER_RAY_SEARCH)) return launch_march_backward_per_ray(m, s);
    int grid = tiled_grid(m);
    if (grid == 0) return cudaSuccess;
    const size_t smem = sizeof(TileShared);
    cudaError_t e = cudaFuncSetAttribute(march_backward_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    march_backward_tiled_kernel<<<grid, kThreads, smem, s>>>(m);
    return cudaGetLastError();
}

}  // namespace rgx
