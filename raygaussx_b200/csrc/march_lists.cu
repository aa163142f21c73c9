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
// CTAs per tile in the forward march and in the replay: each takes an equal share of the tile's rays.  The work
// of a tile is only loosely predicted by the length of its list, so the kernels used to end with a few long
// tiles on otherwise idle SMs (6 % of their time on the 3 M-Gaussian view); smaller units shorten that tail.
#ifndef RGX_TILE_SPLIT
#define RGX_TILE_SPLIT 8          // 3 M-Gaussian step: 1: 440.3 ms, 2: 432.2, 4: 428.5, 8: 427.6 (later: 4: 358.5, 8: 357.5)
#endif
#ifndef RGX_REPLAY_SPLIT
#define RGX_REPLAY_SPLIT 4        // 2: 361.2 ms, 4: 358.5, 8: 358.5
#endif
constexpr int kTileSplit = RGX_TILE_SPLIT;
constexpr int kRaysPerCta = kRaysPerTile / kTileSplit;
constexpr int kReplaySplit = RGX_REPLAY_SPLIT;
constexpr int kRaysPerReplayCta = kRaysPerTile / kReplaySplit;

constexpr int kHitList = 256;      // hits of a slab remembered between the two passes of the backward

// Recording of a forward slab for the backward ("tape"), in ints, 16-byte aligned:
//   [0] tbuffer bits  [1] hit count  [2,3] offset of the ray's next chunk (-1: last)
//   [4, 132) per sample (lane) the sums (sigma, r sigma, g sigma, b sigma) weighted by the Gaussians' responses
//   [132, 132 + hits) sorted slots of the hits in the order they were met
constexpr int kTapeHead = 4 + 4 * kSlab;
constexpr int kTapeBlock = 4096;   // ints a warp reserves at a time; slabs are recorded if kTapeHead + hit cap fits

struct ListShared {
    int next_ray;
    float4 color[kWarps];      // forward: the ray's colour and depth so far (lane 0 of the warp owns it)
    int pend[kWarps][2 * kFan];
    int prim_of[kWarps][kFan];
    WarpStage ws[kWarps];
};

// Where a warp stands on the tape.  Kept in shared memory, not in registers: it is touched once per slab,
// the registers it would take are wanted all the time by the search and the evaluation.
struct TapeState {
    long long off;      // next free int of the warp's current block
    long long head;     // first chunk of the current ray (-1: none yet)
    long long prev;     // latest chunk of the current ray
    int* hits;          // where the current slab's hits go (null: the slab is not recorded)
    int left;           // ints left in the block
    int ok;             // 0: the current ray cannot be recorded (no room)
    unsigned int slabs, nhits;   // recorded by this warp so far (for the backward's choice of kernel)
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
    LeafTest t = test_gaussian(L, r, j, valid, tmin, tmax, tl, COUNT, false);
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
            if (npend >= kFan) {
                const long long c_t = COUNT ? clock64() : 0;
                const bool go = test_pending<COUNT>(L, r, tmin, tmax, pend, npend, lane, tl, leaf);
                if (COUNT) tl.v[C_CYC_WAIT] += clock64() - c_t;       // exact tests and what the caller does with the hits
                if (!go) return;
            }
        }
        if (any_beyond) break;
    }
    while (npend > 0) {
        const long long c_t = COUNT ? clock64() : 0;
        const bool go = test_pending<COUNT>(L, r, tmin, tmax, pend, npend, lane, tl, leaf);
        if (COUNT) tl.v[C_CYC_WAIT] += clock64() - c_t;
        if (!go) return;
    }
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

// A ray stops at the horizon of its lists: counted; in the counting-only variant its number is kept as well, for the
// per-ray search that finishes it (march.cu).
template <int HZ>
__device__ __forceinline__ void hz_note(const MarchLaunch& L, int ray_id) {
    const unsigned int at = atomicAdd(L.hz_count, 1u);
    if (HZ == 2) L.hz_rays[at] = ray_id;
}

// ---------------------------------------------------------------- forward
// HZ: the two-depth variant for forward-only views whose rays end early (binning.cu).  In its first phase
// (L.hz_phase == 1) the tile lists hold only the pairs that begin before L.horizon; a ray that would need more
// -- its next slab reaches past the horizon, or a closest-hit query finds nothing before it, in a tile that has
// pairs beyond (L.tile_more) -- puts its state aside (L.hz_state), flags its tile (L.tile_resume) and stops.
// The second phase (L.hz_phase == 2) has the complete lists of the flagged tiles and takes those rays up where
// they stopped: same slabs, same hits in the same order, same image.
// L.hz_phase == 3 is the first phase without a second one, for recording forwards (training views, whose rays
// are expected to end before the horizon): a ray that would need more is counted and listed (L.hz_rays), marked as
// not recorded, and finished by march_forward_listed_rays_kernel, which the caller launches next.
// HZ = 1: the two phases (L.hz_phase 1 or 2); HZ = 2: counting only (L.hz_phase 3), nothing is put aside.
template <bool COUNT, bool SAVE, int HZ = 0>
__global__ void __launch_bounds__(kThreads, COUNT ? 1 : 4) march_forward_lists_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ ListShared sh;
    __shared__ TapeState tape_state[SAVE ? kWarps : 1];
    constexpr bool save = SAVE;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    WarpStage& ws = sh.ws[warp];
    int* pend = sh.pend[warp];
    const int unit = blockIdx.x / kTileSplit, part = blockIdx.x % kTileSplit;
    const int tile = L.lists.tile_order ? __ldg(&L.lists.tile_order[unit]) : unit;   // longest lists first
    if (HZ == 1 && L.hz_phase == 2 && !L.tile_resume[tile]) return;      // no ray of this tile stopped at the horizon
    // the tile has pairs beyond the horizon that its lists do not hold
    const bool hz_more = HZ != 0 && (HZ == 2 || L.hz_phase == 1) && L.tile_more[tile] != 0;
    const int tile_x = tile % L.lists.tiles_x, tile_y = tile / L.lists.tiles_x;
    const float eps = L.m.transmittance_eps;
    const float bg = L.m.white_background ? 1.0f : 0.0f;
    const SceneBox box = *L.box;
    const TileView tv = tile_view(L.lists, tile);
    Tally tl;
#pragma unroll
    for (int i = 0; i < C_NUM; ++i) tl.v[i] = 0;
    TapeState& tq = tape_state[SAVE ? warp : 0];
    if (tid == 0) sh.next_ray = 0;
    if (save && lane == 0) { tq.off = 0; tq.left = 0; tq.hits = nullptr; tq.slabs = 0u; tq.nhits = 0u; }
    __syncthreads();

    while (true) {
        int ray = 0;
        if (lane == 0) ray = atomicAdd(&sh.next_ray, 1);
        ray = __shfl_sync(kFull, ray, 0);
        if (ray >= kRaysPerCta) break;
        ray += part * kRaysPerCta;
        int px, py;
        if (!ray_pixel(L, tile_x, tile_y, ray, px, py)) continue;
        const int ray_id = py * L.cam.width + px;
        Ray r;
        make_ray(L.cam, px, py, r);
        float tenter, texit;
        clip_scene(box, r, tenter, texit);
        float T = 1.0f;
        if (lane == 0) sh.color[warp] = make_float4(0.f, 0.f, 0.f, 0.f);
        int cursor = 0;
        if (save) {
            if (lane == 0) { tq.head = -1; tq.prev = -1; tq.ok = 1; }
            __syncwarp();
        }
        if (COUNT) tl.v[C_RAYS] += 1;
        // cycle counters of the counting variant: whole ray, closest-hit queries, slab queries (the
        // evaluation of the staged hits is timed inside slab_sums), compositing
        const long long c_ray = COUNT ? clock64() : 0;
        // two-depth variant: 0 = march from the start, 1 = resume at a slab, 2 = resume at the first query,
        // 3 = resume at a query after an empty slab; what was put aside is (tbuffer, T, tenter, mode) + colour
        int hz_mode = 0;
        bool hz_susp = false;
        float4 hz_a = make_float4(0.f, 0.f, 0.f, 0.f);
        if (HZ == 1) {
            if (L.hz_phase == 2) {
                hz_a = L.hz_state[2 * (size_t)ray_id];
                hz_mode = (int)hz_a.w;
                if (hz_mode == 0) continue;                                       // finished in the first phase
                if (hz_mode != 2) {
                    T = hz_a.y;
                    if (lane == 0) sh.color[warp] = L.hz_state[2 * (size_t)ray_id + 1];
                }
            }
        }
        float first;
        if (HZ == 1 && (hz_mode == 1 || hz_mode == 3)) first = hz_a.z;                  // the first hit is known
        else first = closest_in_tile<COUNT>(L, r, tenter, texit, tv, cursor, pend, lane, tl);
        if (COUNT) tl.v[C_CYC_SEEK] += clock64() - c_ray;
        if (HZ && hz_more && !(first < L.horizon)) {                             // nothing before the horizon: ask again later
            hz_susp = true;
            if (lane == 0) {
                if (HZ == 1 && L.hz_phase == 1) {
                    L.hz_state[2 * (size_t)ray_id] = make_float4(tenter, 1.0f, tenter, 2.0f);
                    L.tile_resume[tile] = 1;
                }
                hz_note<HZ>(L, ray_id);
            }
        } else if (first < INFINITY && first < texit) {                           // :249-260
            tenter = first;
            float tbuffer = tenter;
            int slab_index = 0;
            if (HZ == 1 && hz_mode == 1) tbuffer = hz_a.x;
            if (HZ == 1 && hz_mode == 3) {                                             // the query after an empty slab, again
                const float nxt = closest_in_tile<COUNT>(L, r, hz_a.x, texit, tv, cursor, pend, lane, tl);
                tbuffer = nxt < INFINITY ? nxt : texit;                           // nothing further: the loop below does not start
            }
            while (tbuffer < texit && T > eps && slab_index < kMaxSlabs) {        // :266
                SlabPlan p = plan_slab(L.m, tbuffer, T, tenter, texit);
                if (HZ && hz_more && !(p.tmax < L.horizon)) {                        // this slab needs pairs from beyond
                    hz_susp = true;
                    if (lane == 0) {
                        if (HZ == 1 && L.hz_phase == 1) {
                            L.hz_state[2 * (size_t)ray_id] = make_float4(tbuffer, T, tenter, 1.0f);
                            L.hz_state[2 * (size_t)ray_id + 1] = sh.color[warp];
                            L.tile_resume[tile] = 1;
                        }
                        hz_note<HZ>(L, ray_id);
                    }
                    break;
                }
                if (COUNT) tl.v[C_SLABS] += 1;
                ++slab_index;
                if (!p.traced) { tbuffer = __fadd_rn(tbuffer, p.slab); continue; }
                const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
                float s, cr, cg, cb;
                bool overflow;
                // room on the tape for the largest chunk this slab can make; the hits are written there as they
                // are met and the unused rest is handed back
                if (save) {
                    if (lane == 0) {
                        tq.hits = nullptr;
                        if (tq.ok) {
                            const int worst = (kTapeHead + L.m.max_prim_slice + 3) & ~3;
                            if (worst > tq.left && worst <= kTapeBlock) {
                                const unsigned long long o = atomicAdd(L.tape_used, (unsigned long long)kTapeBlock);
                                if ((long long)(o + kTapeBlock) <= L.tape_cap) { tq.off = (long long)o; tq.left = kTapeBlock; }
                            }
                            if (worst <= tq.left) tq.hits = L.tape + tq.off + kTapeHead;
                            else tq.ok = 0;                // no room: the backward will search this ray
                        }
                    }
                    __syncwarp();
                }
                const long long c_q = COUNT ? clock64() : 0;
                int nhit = slab_sums<COUNT, false>(L, L.m, tbuffer, tau, ray_id, slab_index, make_float3(0.f, 0.f, 0.f),
                                                   ws, lane, tl, [&](auto&& leaf) {
                    search_tile<COUNT>(L, r, p.tmin, p.tmax, tv, cursor, pend, lane, tl, leaf);
                }, s, cr, cg, cb, overflow, save ? &tq.hits : nullptr, L.m.max_prim_slice);
                if (COUNT) { tl.v[C_HITS] += nhit; tl.v[C_OVF] += overflow ? 1 : 0; tl.v[C_CYC_SEARCH] += clock64() - c_q; }
                if (save && nhit > 0 && tq.hits) {
                    int* chunk = tq.hits - kTapeHead;
                    reinterpret_cast<float4*>(chunk + 4)[lane] = make_float4(s, cr, cg, cb);
                    __syncwarp();
                    if (lane == 0) {
                        const int need = (kTapeHead + nhit + 3) & ~3;
                        *reinterpret_cast<int4*>(chunk) = make_int4(__float_as_int(tbuffer), nhit, -1, -1);
                        if (tq.prev >= 0)
                            *reinterpret_cast<int2*>(L.tape + tq.prev + 2) = make_int2((int)(tq.off & 0xffffffffll), (int)(tq.off >> 32));
                        if (tq.head < 0) tq.head = tq.off;
                        tq.prev = tq.off;
                        tq.off += need;
                        tq.left -= need;
                        tq.slabs += 1u;
                        tq.nhits += (unsigned int)nhit;
                    }
                    __syncwarp();
                }
                if (nhit == 0) {                                                  // :297-319
                    tbuffer = __fadd_rn(tbuffer, p.slab);
                    const long long c_s = COUNT ? clock64() : 0;
                    float nxt = closest_in_tile<COUNT>(L, r, tbuffer, texit, tv, cursor, pend, lane, tl);
                    if (COUNT) tl.v[C_CYC_SEEK] += clock64() - c_s;
                    if (HZ && hz_more && !(nxt < L.horizon)) {                   // the next hit, if any, is beyond the horizon
                        hz_susp = true;
                        if (lane == 0) {
                            if (HZ == 1 && L.hz_phase == 1) {
                                L.hz_state[2 * (size_t)ray_id] = make_float4(tbuffer, T, tenter, 3.0f);
                                L.hz_state[2 * (size_t)ray_id + 1] = sh.color[warp];
                                L.tile_resume[tile] = 1;
                            }
                            hz_note<HZ>(L, ray_id);
                        }
                        break;
                    }
                    if (!(nxt < INFINITY)) break;
                    tbuffer = nxt;
                    continue;
                }
                if (COUNT) tl.v[C_SLABS_HIT] += 1;
                const long long c_c = COUNT ? clock64() : 0;
                composite_forward_shared(p, tbuffer, tau, eps, lane, s, cr, cg, cb, L.depth != nullptr, T, &sh.color[warp]);
                if (COUNT) tl.v[C_CYC_COMP] += clock64() - c_c;
                tbuffer = __fadd_rn(tbuffer, p.slab);                             // :324
            }
        }
        if (HZ == 2 && hz_susp && save && lane == 0) {             // the backward searches this ray again
            L.ray_head[ray_id] = -2;
            L.tile_unrecorded[tile] = 1;
        }
        if (lane == 0 && !(HZ && hz_susp)) {                                       // :326-339
            const float4 acc = sh.color[warp];
            const RayColor st = {T, acc.x, acc.y, acc.z, acc.w};
            write_ray(L, ray_id, st, bg);
            if (HZ == 1 && L.hz_phase == 1) L.hz_state[2 * (size_t)ray_id] = make_float4(0.f, 0.f, 0.f, 0.f);   // done
            if (save) {
                L.ray_head[ray_id] = tq.ok ? tq.head : -2;
                if (!tq.ok) L.tile_unrecorded[tile] = 1;
            }
        }
        if (COUNT) tl.v[C_CYC_TOTAL] += clock64() - c_ray;
    }
    if (COUNT) flush_tally(L, tl, lane);
    if (save && lane == 0 && tq.slabs) {
        atomicAdd(L.tape_used + 1, (unsigned long long)tq.slabs);
        atomicAdd(L.tape_used + 2, (unsigned long long)tq.nhits);
    }
}

// ---------------------------------------------------------------- backward, by replaying the forward's recording
//
// For rays whose forward was recorded.  Per slab the recording holds the hits and the
// per-sample sums, so what is left is the second pass of the reference's backward
// (cuda_train/backward/gaussians_aabb.cu:354-470): the gradient of every (slab,
// Gaussian) pair.  Here lanes are Gaussians, not samples: a lane takes one hit of the
// slab, walks only the samples that lie inside that Gaussian's truncation ellipsoid
// (a handful of the 32 on average) and keeps the four moment sums in registers -- no
// staging in shared memory and no reduction across lanes.
constexpr int kRun = 4;     // samples per work item of the replay (2: 12.9 ms, 4: 11.1 ms, 8: 11.1 / 7.8 ms on the two test scenes)

constexpr int kBatch = 8;   // slabs of a ray whose hits are worked off together

struct ReplayStage {        // per warp: one group of up to 32 hits
    float4 a[kFan];         // whitened ray point at the reference parameter of the moments, sigma
    float4 b[kFan];         // whitened direction, -
    float4 c[kFan];         // chat_i, tbuffer - reference parameter, first and last sample (as int bits)
    float4 d[kFan];         // the response along the ray as a parabola about the closest approach (march_common.cuh,
                            // eval_forward): -hk q_min, -hk |de|^2, (1 - q_min)/|de|^2, tbuffer - closest approach
    int slot[kFan];
    int upto[kFan];         // inclusive prefix of the number of runs
    int slab[kFan];         // which slab of the batch the hit belongs to
};

template <int NB>
struct ReplayBatchT {       // per warp: up to NB consecutive slabs of the ray
    float2 bg[NB][kSlab];    // per sample: beta, gamma (slab_back_terms)
    float tbuffer[NB];
    float dt[NB];
    long long hits[NB];      // where the slab's hit list starts on the tape
    int upto[NB];            // inclusive prefix of the hit counts
};

template <int NB>
struct ReplayShared {
    int next_ray;
    ReplayBatchT<NB> batch[kWarps];
    ReplayStage stage[kWarps];
};

// Second pass of the backward for the hits of a batch of slabs (see the kernel's comment).
// SINGLE: the batch is one slab (the common case where a slab fills the lanes by itself).
template <bool SINGLE, int NB>
__device__ __forceinline__ void replay_batch(const MarchLaunch& L, const Ray& r, float3 dl, const ReplayBatchT<NB>& bt,
                                             ReplayStage& sp, int nslab, int lane, float tbuffer1, float dt1,
                                             long long hits1, int nhit1) {
    // a single slab's values come in registers (tbuffer1 ...), those of a batch from shared memory
    const int total_hits = SINGLE ? nhit1 : bt.upto[nslab - 1];
    for (int base = 0; base < total_hits; base += kFan) {
        // step 1, one hit per lane: where the ray is inside the Gaussian, cut into runs of kRun samples
        int nitem = 0;
        const int g = base + lane;
        if (g < total_hits) {
            int k = 0;
            if (!SINGLE) {
#pragma unroll
                for (int t = 0; t < NB - 1; ++t) k += (t < nslab - 1 && bt.upto[t] <= g) ? 1 : 0;
            }
            const int j = SINGLE ? L.tape[hits1 + g] : L.tape[bt.hits[k] + (g - (k > 0 ? bt.upto[k - 1] : 0))];
            const float tbuffer = SINGLE ? tbuffer1 : bt.tbuffer[k], dt = SINGLE ? dt1 : bt.dt[k];
            const float inv_dt = __fdividef(1.0f, dt);
            const float tend = __fadd_rn(tbuffer, __fmul_rn(dt, (float)kSlab));
            float3 Oe, de;
            whiten_ray(r, __ldg(&L.g.g0[j]), __ldg(&L.g.g1[j]), __ldg(&L.g.g2[j]), Oe, de);
            const float hk = __ldg(&L.g.hk[j]);
            const float4 c = __ldg(&L.g.rgba[j]);
            const float ci = __fdividef(fmaf(dl.x, c.x, fmaf(dl.y, c.y, __fmul_rn(dl.z, c.z))), c.w);
            // closest approach and half width of the stretch inside the ellipsoid |Oe + t de| < 1
            const float aa = dot3(de, de);
            const float inv_a = __fdividef(1.0f, aa);
            // correctly rounded: the response is evaluated as a parabola about this point, and what the point is
            // off the true closest approach comes back as an unmodelled linear term 2 |de|^2 (tau - tau*) error
            const float tca = __fdiv_rn(-dot3(Oe, de), aa);
            const float3 P = make_float3(fmaf(tca, de.x, Oe.x), fmaf(tca, de.y, Oe.y), fmaf(tca, de.z, Oe.z));
            const float qmin = dot3(P, P);
            const float hw = sqrt_approx(__fmul_rn(fmaxf(1.0f - qmin, 0.f), inv_a));      // only sizes the window of samples
            // samples (s + 1/2) dt inside it, one more on each side against rounding; the test q < 1 decides
            const float x_lo = fmaf(__fadd_rn(__fadd_rn(tca, -hw), -tbuffer), inv_dt, -0.5f);
            const float x_hi = fmaf(__fadd_rn(__fadd_rn(tca, hw), -tbuffer), inv_dt, -0.5f);
            const int s_lo = (int)fminf(fmaxf(ceilf(x_lo) - 1.0f, 0.f), (float)kSlab);
            const int s_hi = (int)fmaxf(fminf(floorf(x_hi) + 1.0f, (float)(kSlab - 1)), -1.f);
            // moments about the closest approach clamped to the slab, so that they stay small
            const float tcr = fminf(fmaxf(tca, tbuffer), tend);
            sp.a[lane] = make_float4(fmaf(tcr, de.x, Oe.x), fmaf(tcr, de.y, Oe.y), fmaf(tcr, de.z, Oe.z), c.w);
            sp.b[lane] = make_float4(de.x, de.y, de.z, 0.f);
            sp.c[lane] = make_float4(ci, __fadd_rn(tbuffer, -tcr), __int_as_float(s_lo), __int_as_float(s_hi));
            sp.d[lane] = make_float4(__fmul_rn(-hk, qmin), __fmul_rn(-hk, aa), __fmul_rn(1.0f - qmin, inv_a),
                                     __fadd_rn(tbuffer, -tca));
            sp.slot[lane] = j;
            if (!SINGLE) sp.slab[lane] = k;
            nitem = s_hi >= s_lo ? (s_hi - s_lo + kRun) / kRun : 0;
        }
        int incl = nitem;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += t;
        }
        const int total = __shfl_sync(kFull, incl, 31);
        sp.upto[lane] = incl;
        __syncwarp();
        // step 2, one run per lane, whichever hit it belongs to: the four moment sums of the run,
        // which share the reference point with the other runs of the hit and so simply add up
        for (int i0 = 0; i0 < total; i0 += kFan) {
            const int i = i0 + lane;
            const bool active = i < total;
            int h = 0;
            float sb = 0.f, n0 = 0.f, n1 = 0.f, n2 = 0.f;
            if (active) {
#pragma unroll
                for (int step = 16; step > 0; step >>= 1)
                    if (sp.upto[h + step - 1] <= i) h += step;          // first hit whose runs end after i
                const float4 C = sp.c[h], D = sp.d[h];
                const int k = SINGLE ? 0 : sp.slab[h];
                const float dt = SINGLE ? dt1 : bt.dt[k];
                const float2* sbg = bt.bg[k];
                const int s_hi = __float_as_int(C.w);
                const int nrun = (s_hi - __float_as_int(C.z) + kRun) / kRun;
                const int s0 = __float_as_int(C.z) + kRun * (i - (sp.upto[h] - nrun));
                // sample position counted from the closest approach (d: the response) and from the reference
                // point of the moments (tc); both advance by dt
                const float x0 = __fmul_rn((float)s0 + 0.5f, dt);
                float d = __fadd_rn(x0, D.w), tc = __fadd_rn(x0, C.y);
#pragma unroll
                for (int q4 = 0; q4 < kRun; ++q4) {
                    const int s = s0 + q4;
                    const float d2 = __fmul_rn(d, d);
                    if (s <= s_hi && d2 < D.z) {
                        const float ex = ex2_approx(fmaf(D.y, d2, D.x));
                        const float2 bg = sbg[s];
                        const float be = bg.x;
                        const float ga = __fmul_rn(ex, fmaf(C.x, be, bg.y));   // g * (alpha + beta*(chat_i - chat_s))
                        const float g1 = __fmul_rn(ga, tc);
                        sb = fmaf(ex, be, sb);
                        n0 = __fadd_rn(n0, ga);
                        n1 = __fadd_rn(n1, g1);
                        n2 = fmaf(g1, tc, n2);
                    }
                    d = __fadd_rn(d, dt);
                    tc = __fadd_rn(tc, dt);
                }
            }
            // runs of one hit sit in neighbouring lanes (at most 32 / kRun of them): add them up so that
            // the Gaussian's row gets one update per hit, not one per run
            const int seg = active ? h : -1 - lane;
#pragma unroll
            for (int d = 1; d < kSlab / kRun; d <<= 1) {
                const int seg_o = __shfl_down_sync(kFull, seg, d);
                const float o_sb = __shfl_down_sync(kFull, sb, d), o_n0 = __shfl_down_sync(kFull, n0, d),
                            o_n1 = __shfl_down_sync(kFull, n1, d), o_n2 = __shfl_down_sync(kFull, n2, d);
                if (lane + d < 32 && seg_o == seg) {
                    sb = __fadd_rn(sb, o_sb); n0 = __fadd_rn(n0, o_n0); n1 = __fadd_rn(n1, o_n1); n2 = __fadd_rn(n2, o_n2);
                }
            }
            const int seg_prev = __shfl_up_sync(kFull, seg, 1);
            const bool first = lane == 0 || seg_prev != seg;
            if (active && first && (sb != 0.f || n0 != 0.f || n1 != 0.f || n2 != 0.f)) {
                const float4 A = sp.a[h];
                emit_global(L, dl, sp.slot[h], expand_gradient(A.w, A, sp.b[h], sb, n0, n1, n2), blockIdx.x / kReplaySplit);
            }
        }
        __syncwarp();                      // the next group reuses the staging arrays
    }
}

// NB: slabs batched.  1 where slabs fill the lanes by themselves (fewer registers, one more CTA per SM).
template <int NB>
__global__ void __launch_bounds__(kThreads) march_backward_replay_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ ReplayShared<NB> sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit = blockIdx.x / kReplaySplit, part = blockIdx.x % kReplaySplit;
    const int tile = L.replay_order ? __ldg(&L.replay_order[unit]) : unit;
    const int tile_x = tile % L.lists.tiles_x, tile_y = tile / L.lists.tiles_x;
    const float eps = L.m.transmittance_eps;
    const SceneBox box = *L.box;
    ReplayBatchT<NB>& bt = sh.batch[warp];
    ReplayStage& sp = sh.stage[warp];
    if (tid == 0) sh.next_ray = 0;
    __syncthreads();

    while (true) {
        int ray = 0;
        if (lane == 0) ray = atomicAdd(&sh.next_ray, 1);
        ray = __shfl_sync(kFull, ray, 0);
        if (ray >= kRaysPerReplayCta) break;
        ray += part * kRaysPerReplayCta;
        int px, py;
        if (!ray_pixel(L, tile_x, tile_y, ray, px, py)) continue;
        const int ray_id = py * L.cam.width + px;
        long long off = L.ray_head[ray_id];
        if (off < 0) continue;                     // -1: the ray met nothing; -2: not recorded, left to the search kernel
        Ray r;
        make_ray(L.cam, px, py, r);
        float tenter, texit;
        clip_scene(box, r, tenter, texit);
        const float3 dl = make_float3(L.dl_drgb[3 * (size_t)ray_id], L.dl_drgb[3 * (size_t)ray_id + 1],
                                      L.dl_drgb[3 * (size_t)ray_id + 2]);
        float D = fmaf(dl.x, L.rgb_in[3 * (size_t)ray_id],
                       fmaf(dl.y, L.rgb_in[3 * (size_t)ray_id + 1], __fmul_rn(dl.z, L.rgb_in[3 * (size_t)ray_id + 2])));
        float T = 1.0f;
        int nslab = 0, nhits = 0;
        while (off >= 0) {
            // first pass of a slab, from the recording: transmittance and the per-sample terms
            const int4 hd = *reinterpret_cast<const int4*>(L.tape + off);
            const float tbuffer = __int_as_float(hd.x);
            const int nhit = hd.y;
            const float4 sums = reinterpret_cast<const float4*>(L.tape + off + 4)[lane];
            const long long hits_at = off + kTapeHead;
            off = ((long long)hd.w << 32) | (unsigned int)hd.z;
            // same step size as the forward: T is rebuilt from the recorded sums bit for bit
            const SlabPlan p = plan_slab(L.m, tbuffer, T, tbuffer, texit);
            const float dc = fmaf(dl.x, sums.y, fmaf(dl.y, sums.z, __fmul_rn(dl.z, sums.w)));
            const SlabBackTerms terms = slab_back_terms(sums.x, dc, p.dt, T, D, eps, lane);
            D = __fadd_rn(D, -terms.d_total);
            T = slab_exit_T(terms.tr, eps);
            bt.bg[nslab][lane] = make_float2(terms.beta, terms.gamma);
            nhits += nhit;
            if (lane == 0) { bt.tbuffer[nslab] = tbuffer; bt.dt[nslab] = p.dt; bt.hits[nslab] = hits_at; bt.upto[nslab] = nhits; }
            ++nslab;
            if (NB == 1 || nhits >= kFan || nslab == NB || off < 0) {   // enough hits to fill the lanes, or nothing more to wait for
                __syncwarp();
                if (NB == 1 || nslab == 1) replay_batch<true>(L, r, dl, bt, sp, 1, lane, tbuffer, p.dt, hits_at, nhit);
                else replay_batch<false>(L, r, dl, bt, sp, nslab, lane, 0.f, 0.f, 0, 0);
                nslab = 0;
                nhits = 0;
            }
        }
    }
}

// ---------------------------------------------------------------- backward, by searching again
// For rays without a recording: all of them when the forward did not record, else only those
// it could not record (ray_head == -2).
__global__ void __launch_bounds__(kThreads) march_backward_lists_kernel(const __grid_constant__ MarchLaunch L) {
    __shared__ ListShared sh;
    __shared__ int hit_lists[kWarps][kHitList];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    WarpStage& ws = sh.ws[warp];
    int* pend = sh.pend[warp];
    const int tile = L.lists.tile_order ? __ldg(&L.lists.tile_order[blockIdx.x]) : blockIdx.x;
    if (L.tape && !L.tile_unrecorded[tile]) return;             // every ray of the tile was recorded: the replay kernel's
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
        if (L.tape && L.ray_head[ray_id] != -2) continue;       // recorded: the replay kernel's
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
                                              u0, u1, overflow, &hits, kHitList);
            if (nhit == 0) {
                tbuffer = __fadd_rn(tbuffer, p.slab);
                float nxt = closest_in_tile<false>(L, r, tbuffer, texit, tv, cursor, pend, lane, tl);
                if (!(nxt < INFINITY)) break;
                tbuffer = nxt;
                continue;
            }
            SlabBackTerms bt = slab_back_terms(s, dc, p.dt, T, D, eps, lane);
            // pass 2: the hits again -- from the remembered list when it held them all, else by a second query
            auto emit = [&](int j, const GaussGrad& g) { emit_global(L, dl, j, g, blockIdx.x); };
            if (nhit <= kHitList) {
                __syncwarp();
                slab_gradients(L, L.m, r, p, tbuffer, tau, dl, bt.beta, bt.gamma, ws, sh.prim_of[warp], lane,
                               [&](auto&& leaf) {
                                   for (int base = 0; base < nhit; base += kFan) {
                                       const bool valid = base + lane < nhit;
                                       const int j = valid ? hits[base + lane] : 0;
                                       LeafTest t = test_gaussian(L, r, j, valid, p.tmin, p.tmax, tl, false, false);
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
    const int ctas = grid * kTileSplit;
    if (m.hz_phase == 3) {
        if (save) note_launch(), march_forward_lists_kernel<false, true, 2><<<ctas, kThreads, 0, s>>>(m);
        else note_launch(), march_forward_lists_kernel<false, false, 2><<<ctas, kThreads, 0, s>>>(m);
        return cudaGetLastError();
    }
    if (m.hz_phase != 0) {
        if (save) note_launch(), march_forward_lists_kernel<false, true, 1><<<ctas, kThreads, 0, s>>>(m);
        else note_launch(), march_forward_lists_kernel<false, false, 1><<<ctas, kThreads, 0, s>>>(m);
        return cudaGetLastError();
    }
    if (count && save) note_launch(), march_forward_lists_kernel<true, true><<<ctas, kThreads, 0, s>>>(m);
    else if (count) note_launch(), march_forward_lists_kernel<true, false><<<ctas, kThreads, 0, s>>>(m);
    else if (save) note_launch(), march_forward_lists_kernel<false, true><<<ctas, kThreads, 0, s>>>(m);
    else note_launch(), march_forward_lists_kernel<false, false><<<ctas, kThreads, 0, s>>>(m);
    return cudaGetLastError();
}

cudaError_t launch_march_backward_search(const MarchLaunch& m, cudaStream_t s) {
    if (!use_lists(m)) return launch_march_backward_per_ray(m, s);
    const int grid = m.lists.tiles_x * m.lists.tiles_y;
    if (grid <= 0) return cudaSuccess;
    note_launch(), march_backward_lists_kernel<<<grid, kThreads, 0, s>>>(m);   // a CTA whose tile was recorded completely returns at once
    return cudaGetLastError();
}

cudaError_t launch_march_backward_replay(const MarchLaunch& m, cudaStream_t s) {
    if (!use_lists(m) || !m.tape) return cudaSuccess;
    const int grid = m.lists.tiles_x * m.lists.tiles_y;
    if (grid <= 0) return cudaSuccess;
    if (m.replay_batched) note_launch(), march_backward_replay_kernel<kBatch><<<grid * kReplaySplit, kThreads, 0, s>>>(m);
    else note_launch(), march_backward_replay_kernel<1><<<grid * kReplaySplit, kThreads, 0, s>>>(m);
    return cudaGetLastError();
}

}  // namespace rgx
