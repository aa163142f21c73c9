// Forward and backward ray march over per-view tile lists: the default path.
//
// binning.cu leaves, for every 16x16-pixel tile of the view, a front-to-back list
// of the Gaussians that any ray of the tile can meet, each with the range of
// distances from the eye that its box spans, plus a (nearest near, farthest far)
// summary per 32 entries.  A CTA owns a tile; its eight warps take the tile's
// rays one at a time (one warp marches one ray, lanes = samples of a slab, as in
// march.cu).  A query over [tmin,tmax] looks at 32 block summaries per step, opens
// only the blocks whose range overlaps the query, filters their entries by range,
// compacts the survivors into full groups of 32 and runs the exact per-ray test
// on those.  A per-ray cursor skips the blocks the ray has left behind for good.
// There is no hierarchy search, no CTA-wide barrier and no waiting between rays.
//
// The list is a superset of every hit set and the deciding test is the per-ray one
// of march_common.cuh, so hit sets equal those of the per-ray and exhaustive
// variants; hits are met in list order (near distance, then sorted slot), the same
// in the forward and in both passes of the backward.
//
// Reference semantics: cuda_train/forward/gaussians_aabb.cu:205-340 and
// cuda_train/backward/gaussians_aabb.cu:209-497 (see march_common.cuh).
#include "march_common.cuh"

namespace rgx {

namespace {

constexpr int kRaysPerTile = kBinTile * kBinTile;
constexpr int kThreads = kWarps * 32;

constexpr int kHitList = 256;      // hits of a slab remembered between the two passes of the backward

struct ListShared {
    int next_ray;
    int pend[kWarps][2 * kFan];
    int prim_of[kWarps][kFan];
    WarpStage ws[kWarps];
};

struct TileView {      // one tile's list
    const int* id;
    const float2* range;
    const float2* blk;
    int nblk;
};

__device__ __forceinline__ TileView tile_view(const TileLists& l, int tile) {
    TileView v;
    const int begin = __ldg(&l.tile_pbegin[tile]);
    v.id = l.ent_id + begin;
    v.range = l.ent_range + begin;
    v.blk = l.blk + begin / 32;
    v.nblk = (__ldg(&l.tile_cnt[tile]) + 31) / 32;
    return v;
}

// Runs the exact test on the first min(npend, 32) pending candidates and hands them to leaf.
template <bool COUNT, class LeafFn>
__device__ __forceinline__ bool test_pending(const MarchLaunch& L, const Ray& r, float tmin, float tmax, int* pend,
                                             int& npend, int lane, Tally& tl, LeafFn&& leaf) {
    const bool valid = lane < npend;
    const int j = valid ? pend[lane] : 0;
    LeafTest t = test_gaussian(L, r, j, valid, tmin, tmax, tl, COUNT);
    const bool go = leaf(t, j);
    const int moved = (lane + kFan < npend) ? pend[lane + kFan] : 0;
    __syncwarp();
    pend[lane] = moved;
    npend = npend > kFan ? npend - kFan : 0;
    __syncwarp();
    return go;
}

// Any-hit query over a tile list.  `cursor` is the ray's first block that may still
// matter; it only moves forward because a ray's tmin never decreases.
template <bool COUNT, class LeafFn>
__device__ __forceinline__ void search_tile(const MarchLaunch& L, const Ray& r, float tmin, float tmax,
                                            const TileView& tv, int& cursor, int* pend, int lane, Tally& tl,
                                            LeafFn&& leaf) {
    int npend = 0;
    bool advancing = true;
    for (int b0 = cursor; b0 < tv.nblk; b0 += kFan) {
        const int bi = b0 + lane;
        const bool valid = bi < tv.nblk;
        const float2 s = valid ? __ldg(&tv.blk[bi]) : make_float2(INFINITY, -INFINITY);
        const bool reaches = valid && s.y >= tmin;          // something in the block extends to tmin or beyond
        const bool beyond = valid && s.x > tmax;            // the block, and every later one, starts after tmax
        unsigned live = __ballot_sync(kFull, reaches && !beyond);
        const unsigned any_beyond = __ballot_sync(kFull, beyond);
        if (advancing) {
            const unsigned alive = __ballot_sync(kFull, reaches);
            if (alive == 0u) cursor = min(b0 + kFan, tv.nblk);
            else { cursor = b0 + __ffs(alive) - 1; advancing = false; }
        }
        while (live) {
            const int bb = b0 + __ffs(live) - 1;
            live &= live - 1;
            const int k = bb * kFan + lane;
            const float2 rg = __ldg(&tv.range[k]);
            const bool pass = rg.x <= tmax && rg.y >= tmin;
            const unsigned m = __ballot_sync(kFull, pass);
            if (pass) pend[npend + __popc(m & ((1u << lane) - 1u))] = __ldg(&tv.id[k]);
            npend += __popc(m);
            if (COUNT) tl.v[C_CANDS] += 32;
            __syncwarp();
            if (npend >= kFan && !test_pending<COUNT>(L, r, tmin, tmax, pend, npend, lane, tl, leaf)) return;
        }
        if (any_beyond) break;
    }
    while (npend > 0)
        if (!test_pending<COUNT>(L, r, tmin, tmax, pend, npend, lane, tl, leaf)) return;
}

// Closest hit over [tmin,tmax] in a tile list, +inf on a miss.
template <bool COUNT>
__device__ __forceinline__ float closest_in_tile(const MarchLaunch& L, const Ray& r, float tmin, float tmax,
                                                 const TileView& tv, int& cursor, int* pend, int lane, Tally& tl) {
    float best = INFINITY;
    if (COUNT) tl.v[C_CLOSEST] += 1;
    if (!(tmin <= tmax)) return best;
    int npend = 0;
    bool advancing = true, done = false;
    auto leaf = [&](const LeafTest& t, int) {
        best = fminf(best, warp_min_f(t.hit ? t.t_hit : INFINITY));
        return true;
    };
    for (int b0 = cursor; b0 < tv.nblk && !done; b0 += kFan) {
        const int bi = b0 + lane;
        const bool valid = bi < tv.nblk;
        const float2 s = valid ? __ldg(&tv.blk[bi]) : make_float2(INFINITY, -INFINITY);
        const bool reaches = valid && s.y >= tmin;
        unsigned live = __ballot_sync(kFull, reaches && s.x <= tmax);
        const unsigned any_beyond = __ballot_sync(kFull, valid && s.x > tmax);
        if (advancing) {
            const unsigned alive = __ballot_sync(kFull, reaches);
            if (alive == 0u) cursor = min(b0 + kFan, tv.nblk);
            else { cursor = b0 + __ffs(alive) - 1; advancing = false; }
        }
        while (live) {
            const int src = __ffs(live) - 1;
            live &= live - 1;
            // entries are sorted by near distance: nothing from here on can start before `best`
            if (__shfl_sync(kFull, s.x, src) > best) { done = true; break; }
            const int k = (b0 + src) * kFan + lane;
            const float2 rg = __ldg(&tv.range[k]);
            const bool pass = rg.x <= fminf(tmax, best) && rg.y >= tmin;
            const unsigned m = __ballot_sync(kFull, pass);
            if (pass) pend[npend + __popc(m & ((1u << lane) - 1u))] = __ldg(&tv.id[k]);
            npend += __popc(m);
            if (COUNT) tl.v[C_CANDS] += 32;
            __syncwarp();
            if (npend >= kFan) test_pending<COUNT>(L, r, tmin, fminf(tmax, best), pend, npend, lane, tl, leaf);
        }
        // do not run far ahead with untested candidates: they may already hold the answer
        while (npend > 0) test_pending<COUNT>(L, r, tmin, fminf(tmax, best), pend, npend, lane, tl, leaf);
        if (any_beyond) break;
    }
    return best;
}

// pixel of the tile's ray number `ray` (row-major inside the tile)
__device__ __forceinline__ bool ray_pixel(const MarchLaunch& L, int tile_x, int tile_y, int ray, int& px, int& py) {
    px = tile_x * kBinTile + ray % kBinTile;
    py = (L.lists.ty_first + tile_y) * kBinTile + ray / kBinTile;
    return px < L.cam.width && py >= L.m.row_begin && py < L.m.row_end;
}

// ---------------------------------------------------------------- forward
template <bool COUNT, bool SAVE>
__global__ void __launch_bounds__(kThreads) march_forward_lists_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ ListShared sh;
    __shared__ int hit_lists[SAVE ? kWarps : 1][SAVE ? kHitList : 1];
    constexpr bool save = SAVE;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    WarpStage& ws = sh.ws[warp];
    int* pend = sh.pend[warp];
    const int tile = blockIdx.x;
    const int tile_x = tile % L.lists.tiles_x, tile_y = tile / L.lists.tiles_x;
    const float eps = L.m.transmittance_eps;
    const float bg = L.m.white_background ? 1.0f : 0.0f;
    const SceneBox box = *L.box;
    const TileView tv = tile_view(L.lists, tile);
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;
    if (tid == 0) sh.next_ray = 0;
    __syncthreads();

    while (true) {
        int ray = 0;
        if (lane == 0) ray = atomicAdd(&sh.next_ray, 1);
        ray = __shfl_sync(kFull, ray, 0);
        if (ray >= kRaysPerTile) break;
        int px, py;
        if (!ray_pixel(L, tile_x, tile_y, ray, px, py)) continue;
        const int ray_id = py * L.cam.width + px;
        Ray r;
        make_ray(L.cam, px, py, r);
        float tenter, texit;
        clip_scene(box, r, tenter, texit);
        RayColor st = {1.0f, 0.f, 0.f, 0.f, 0.f};
        int cursor = 0;
        long long tape_head = -1, tape_prev = -1;    // first and latest chunk of this ray on the tape
        bool tape_ok = true;
        if (COUNT) tl.v[C_RAYS] += 1;
        float first = closest_in_tile<COUNT>(L, r, tenter, texit, tv, cursor, pend, lane, tl);
        if (first < INFINITY && first < texit) {                                  // :249-260
            tenter = first;
            float tbuffer = tenter;
            int slab_index = 0;
            while (tbuffer < texit && st.T > eps && slab_index < kMaxSlabs) {     // :266
                SlabPlan p = plan_slab(L.m, tbuffer, st.T, tenter, texit);
                if (COUNT) tl.v[C_SLABS] += 1;
                ++slab_index;
                if (!p.traced) { tbuffer = __fadd_rn(tbuffer, p.slab); continue; }
                const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
                float s, cr, cg, cb;
                bool overflow;
                int* hits = hit_lists[SAVE ? warp : 0];
                int nhit = slab_sums<COUNT, false>(L, L.m, tbuffer, tau, ray_id, slab_index, make_float3(0.f, 0.f, 0.f),
                                                   ws, lane, tl, [&](auto&& leaf) {
                    search_tile<COUNT>(L, r, p.tmin, p.tmax, tv, cursor, pend, lane, tl, leaf);
                }, s, cr, cg, cb, overflow, save ? hits : nullptr, kHitList);
                if (COUNT) { tl.v[C_HITS] += nhit; tl.v[C_OVF] += overflow ? 1 : 0; }
                if (save && nhit > 0 && tape_ok) {
                    // one chunk per slab with hits: [tbuffer, count, next lo, next hi, slots...]
                    long long off = -1;
                    if (nhit <= kHitList) {
                        unsigned long long o = 0;
                        if (lane == 0) o = atomicAdd(L.tape_used, (unsigned long long)(4 + nhit));
                        o = __shfl_sync(kFull, o, 0);
                        if ((long long)(o + 4 + nhit) <= L.tape_cap) off = (long long)o;
                    }
                    if (off < 0) tape_ok = false;          // no room (or too many hits): the backward will search this ray
                    else {
                        __syncwarp();
                        if (lane == 0) {
                            L.tape[off] = __float_as_int(tbuffer); L.tape[off + 1] = nhit;
                            L.tape[off + 2] = -1; L.tape[off + 3] = -1;
                            if (tape_prev >= 0) { L.tape[tape_prev + 2] = (int)(off & 0xffffffffll); L.tape[tape_prev + 3] = (int)(off >> 32); }
                        }
                        for (int i = lane; i < nhit; i += 32) L.tape[off + 4 + i] = hits[i];
                        if (tape_head < 0) tape_head = off;
                        tape_prev = off;
                        __syncwarp();
                    }
                }
                if (nhit == 0) {                                                  // :297-319
                    tbuffer = __fadd_rn(tbuffer, p.slab);
                    float nxt = closest_in_tile<COUNT>(L, r, tbuffer, texit, tv, cursor, pend, lane, tl);
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
            L.rgb[3 * (size_t)ray_id] = fmaf(st.T, bg, st.Cr);
            L.rgb[3 * (size_t)ray_id + 1] = fmaf(st.T, bg, st.Cg);
            L.rgb[3 * (size_t)ray_id + 2] = fmaf(st.T, bg, st.Cb);
            if (L.alpha) L.alpha[ray_id] = 1.0f - st.T;
            if (L.depth) L.depth[ray_id] = st.depth;
            if (save) L.ray_head[ray_id] = tape_ok ? tape_head : -2;
        }
    }
    if (COUNT) flush_tally(L, tl, lane);
}

// ---------------------------------------------------------------- backward
// TAPE = true: rays whose forward was recorded, replayed from the tape, no search code at all.
// TAPE = false: rays without a recording (all of them when nothing was recorded), by searching again.
template <bool TAPE>
__global__ void __launch_bounds__(kThreads) march_backward_lists_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ ListShared sh;
    __shared__ int hit_lists[kWarps][kHitList];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    WarpStage& ws = sh.ws[warp];
    int* pend = sh.pend[warp];
    const int tile = blockIdx.x;
    const int tile_x = tile % L.lists.tiles_x, tile_y = tile / L.lists.tiles_x;
    const float eps = L.m.transmittance_eps;
    const SceneBox box = *L.box;
    const TileView tv = tile_view(L.lists, tile);
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;
    if (tid == 0) sh.next_ray = 0;
    __syncthreads();

    while (true) {
        int ray = 0;
        if (lane == 0) ray = atomicAdd(&sh.next_ray, 1);
        ray = __shfl_sync(kFull, ray, 0);
        if (ray >= kRaysPerTile) break;
        int px, py;
        if (!ray_pixel(L, tile_x, tile_y, ray, px, py)) continue;
        const int ray_id = py * L.cam.width + px;
        Ray r;
        make_ray(L.cam, px, py, r);
        float tenter, texit;
        clip_scene(box, r, tenter, texit);
        int cursor = 0;
        const float3 dl = make_float3(L.dl_drgb[3 * (size_t)ray_id], L.dl_drgb[3 * (size_t)ray_id + 1],
                                      L.dl_drgb[3 * (size_t)ray_id + 2]);
        float D = fmaf(dl.x, L.rgb_in[3 * (size_t)ray_id],
                       fmaf(dl.y, L.rgb_in[3 * (size_t)ray_id + 1], __fmul_rn(dl.z, L.rgb_in[3 * (size_t)ray_id + 2])));
        float T = 1.0f;
        const long long head = L.tape ? L.ray_head[ray_id] : -2;
        if (TAPE != (head != -2)) continue;
        if (TAPE) {
            // The forward left this ray's slabs on the tape: same hits in the same order, so the sums, the
            // transmittance and with it the step sizes come out bit for bit as in the forward -- no search.
            long long off = head;
            int* hits = hit_lists[warp];
            while (off >= 0) {
                const float tbuffer = __int_as_float(L.tape[off]);
                const int nhit = L.tape[off + 1];
                const long long next = ((long long)L.tape[off + 3] << 32) | (unsigned int)L.tape[off + 2];
                for (int i = lane; i < nhit; i += 32) hits[i] = L.tape[off + 4 + i];
                __syncwarp();
                SlabPlan p = plan_slab(L.m, tbuffer, T, tbuffer, texit);
                const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
                auto replay = [&](auto&& leaf) {
                    for (int base = 0; base < nhit; base += kFan) {
                        const bool valid = base + lane < nhit;
                        const int j = valid ? hits[base + lane] : 0;
                        LeafTest t;
                        t.hit = valid;
                        t.t_hit = 0.f;
                        if (valid) whiten_ray(r, __ldg(&L.g.g0[j]), __ldg(&L.g.g1[j]), __ldg(&L.g.g2[j]), t.Oe, t.de);
                        if (!leaf(t, j)) return;
                    }
                };
                float s, dc, u0, u1;
                bool overflow;
                slab_sums<false, true>(L, L.m, tbuffer, tau, ray_id, 0, dl, ws, lane, tl, replay, s, dc, u0, u1, overflow);
                SlabBackTerms bt = slab_back_terms(s, dc, p.dt, T, D, eps, lane);
                slab_gradients(L, L.m, r, p, tbuffer, tau, dl, bt.beta, bt.gamma, ws, sh.prim_of[warp], lane, replay,
                               [&](int j, const GaussGrad& g) { emit_global(L, dl, j, g); });
                D = __fadd_rn(D, -bt.d_total);
                T = slab_exit_T(bt.tr, eps);
                off = next;
                __syncwarp();
            }
            continue;
        }
        if constexpr (!TAPE) {
        float first = closest_in_tile<false>(L, r, tenter, texit, tv, cursor, pend, lane, tl);
        if (!(first < INFINITY && first < texit)) continue;                       // backward .cu:249-254
        tenter = first;
        float tbuffer = tenter;
        int slab_index = 0;
        while (tbuffer < texit && T > eps && slab_index < kMaxSlabs) {
            SlabPlan p = plan_slab(L.m, tbuffer, T, tenter, texit);
            ++slab_index;
            if (!p.traced) { tbuffer = __fadd_rn(tbuffer, p.slab); continue; }
            const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
            auto enumerate = [&](auto&& leaf) { search_tile<false>(L, r, p.tmin, p.tmax, tv, cursor, pend, lane, tl, leaf); };
            float s, dc, u0, u1;
            bool overflow;
            int* hits = hit_lists[warp];
            int nhit = slab_sums<false, true>(L, L.m, tbuffer, tau, ray_id, slab_index, dl, ws, lane, tl, enumerate, s, dc,
                                              u0, u1, overflow, hits, kHitList);
            if (nhit == 0) {
                tbuffer = __fadd_rn(tbuffer, p.slab);
                float nxt = closest_in_tile<false>(L, r, tbuffer, texit, tv, cursor, pend, lane, tl);
                if (!(nxt < INFINITY)) break;
                tbuffer = nxt;
                continue;
            }
            SlabBackTerms bt = slab_back_terms(s, dc, p.dt, T, D, eps, lane);
            // pass 2: the hits again -- from the remembered list when it held them all, else by a second query
            auto emit = [&](int j, const GaussGrad& g) { emit_global(L, dl, j, g); };
            if (nhit <= kHitList) {
                __syncwarp();
                slab_gradients(L, L.m, r, p, tbuffer, tau, dl, bt.beta, bt.gamma, ws, sh.prim_of[warp], lane,
                               [&](auto&& leaf) {
                                   for (int base = 0; base < nhit; base += kFan) {
                                       const bool valid = base + lane < nhit;
                                       const int j = valid ? hits[base + lane] : 0;
                                       LeafTest t = test_gaussian(L, r, j, valid, p.tmin, p.tmax, tl, false);
                                       if (!leaf(t, j)) return;
                                   }
                               }, emit);
            } else {
                slab_gradients(L, L.m, r, p, tbuffer, tau, dl, bt.beta, bt.gamma, ws, sh.prim_of[warp], lane, enumerate, emit);
            }
            D = __fadd_rn(D, -bt.d_total);
            T = slab_exit_T(bt.tr, eps);
            tbuffer = __fadd_rn(tbuffer, p.slab);
        }
        }   // !TAPE
    }
}

}  // namespace

cudaError_t launch_march_forward_per_ray(const MarchLaunch& m, cudaStream_t s);
cudaError_t launch_march_backward_per_ray(const MarchLaunch& m, cudaStream_t s);

static bool use_lists(const MarchLaunch& m) {
    return !(m.m.flags & (RGX_FLAG_BRUTE_FORCE | RGX_FLAG_PER_RAY_SEARCH)) && m.lists.ent_id != nullptr && m.g.n > 0;
}

cudaError_t launch_march_forward(const MarchLaunch& m, cudaStream_t s) {
    if (!use_lists(m)) return launch_march_forward_per_ray(m, s);
    const int grid = m.lists.tiles_x * m.lists.tiles_y;
    if (grid <= 0) return cudaSuccess;
    const bool count = (m.m.flags & RGX_FLAG_COUNT_WORK) != 0, save = m.tape != nullptr;
    if (count && save) march_forward_lists_kernel<true, true><<<grid, kThreads, 0, s>>>(m);
    else if (count) march_forward_lists_kernel<true, false><<<grid, kThreads, 0, s>>>(m);
    else if (save) march_forward_lists_kernel<false, true><<<grid, kThreads, 0, s>>>(m);
    else march_forward_lists_kernel<false, false><<<grid, kThreads, 0, s>>>(m);
    return cudaGetLastError();
}

cudaError_t launch_march_backward(const MarchLaunch& m, cudaStream_t s) {
    if (!use_lists(m)) return launch_march_backward_per_ray(m, s);
    const int grid = m.lists.tiles_x * m.lists.tiles_y;
    if (grid <= 0) return cudaSuccess;
    if (m.tape) march_backward_lists_kernel<true><<<grid, kThreads, 0, s>>>(m);     // recorded rays
    march_backward_lists_kernel<false><<<grid, kThreads, 0, s>>>(m);               // the others (a quick no-op per recorded ray)
    return cudaGetLastError();
}

}  // namespace rgx
