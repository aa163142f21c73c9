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
#include "rgx_internal.cuh"
#include "device_math.cuh"

namespace rgx {

namespace {

constexpr int kWarps = 8;
constexpr int kStack = 192;
constexpr int kStage = 64;
constexpr unsigned kFull = 0xffffffffu;
constexpr int kTile = 8;   // CTA = 8x8 pixels; warp w marches column w of the tile
constexpr int kMaxSlabs = 1 << 22;   // hard bound on slab iterations per ray

struct WarpShared {
    float4 recA[kStage];
    float4 recB[kStage];
    float4 recC[kStage];
    uint32_t stack[kStack];
    float stack_t[kStack];
};

struct Ray {
    float3 o, d, inv;
};

struct Tally {   // per-warp work counters (uniform across lanes)
    unsigned long long v[12];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(kFull, v, o));
    return v;
}
__device__ __forceinline__ float warp_min_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}
// inclusive prefix sum over lanes
__device__ __forceinline__ float warp_scan(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float t = __shfl_up_sync(kFull, v, o);
        if (lane >= o) v = __fadd_rn(v, t);
    }
    return v;
}
__device__ __forceinline__ float exp_neg(float x) {   // exp(-x), x >= 0
    return ex2_approx(__fmul_rn(x, -1.4426950408889634f));
}

// cuda_train/forward/gaussians_aabb.cu:95-110
__device__ __forceinline__ void make_ray(const rgx_camera& c, int px, int py, Ray& r) {
    float ix = __fdiv_rn((float)px + 0.5f, (float)c.width);
    float iy = __fdiv_rn((float)py + 0.5f, (float)c.height);
    float a = __fmul_rn(__fmul_rn(2.0f, ix - c.pp[0]), c.tan_half_fov[0]);
    float b = __fmul_rn(__fmul_rn(2.0f, iy - c.pp[1]), c.tan_half_fov[1]);
    float3 d = make_float3(__fadd_rn(__fadd_rn(__fmul_rn(a, c.u[0]), __fmul_rn(b, c.v[0])), c.w[0]),
                           __fadd_rn(__fadd_rn(__fmul_rn(a, c.u[1]), __fmul_rn(b, c.v[1])), c.w[1]),
                           __fadd_rn(__fadd_rn(__fmul_rn(a, c.u[2]), __fmul_rn(b, c.v[2])), c.w[2]));
    float inv_len = __fdiv_rn(1.0f, __fsqrt_rn(dot3(d, d)));
    r.d = make_float3(__fmul_rn(d.x, inv_len), __fmul_rn(d.y, inv_len), __fmul_rn(d.z, inv_len));
    r.o = make_float3(c.eye[0], c.eye[1], c.eye[2]);
    r.inv = make_float3(__frcp_rn(r.d.x), __frcp_rn(r.d.y), __frcp_rn(r.d.z));
}

// Ray/box overlap restricted to [tmin,tmax].  The near/far planes are chosen by the
// sign of the direction (no min/max swap), so an inverted box is never hit, and
// the result is monotone in the box: a box containing a hit box is hit.
__device__ __forceinline__ bool box_hit(const Ray& r, float2 bx, float2 by, float2 bz, float tmin, float tmax,
                                        float& tnear) {
    float x0 = __fmul_rn(bx.x - r.o.x, r.inv.x), x1 = __fmul_rn(bx.y - r.o.x, r.inv.x);
    float y0 = __fmul_rn(by.x - r.o.y, r.inv.y), y1 = __fmul_rn(by.y - r.o.y, r.inv.y);
    float z0 = __fmul_rn(bz.x - r.o.z, r.inv.z), z1 = __fmul_rn(bz.y - r.o.z, r.inv.z);
    bool px = r.inv.x >= 0.f, py = r.inv.y >= 0.f, pz = r.inv.z >= 0.f;
    float nx = px ? x0 : x1, fx = px ? x1 : x0;
    float ny = py ? y0 : y1, fy = py ? y1 : y0;
    float nz = pz ? z0 : z1, fz = pz ? z1 : z0;
    tnear = fmaxf(fmaxf(nx, ny), fmaxf(nz, tmin));
    float tfar = fminf(fminf(fx, fy), fminf(fz, tmax));
    return tnear <= tfar;
}

// Interval of the ray inside the truncation ellipsoid
// (cuda_train/forward/gaussians_aabb.cu:43-91 with M = S^-1 R^T / k folded into g0..g2).
__device__ __forceinline__ bool ellipsoid_interval(const Ray& r, float4 g0, float4 g1, float4 g2, float3& Oe,
                                                   float3& de, float& r1, float& r2) {
    float3 O = make_float3(r.o.x - g0.x, r.o.y - g0.y, r.o.z - g0.z);
    Oe.x = fmaf(g0.w, O.x, fmaf(g1.x, O.y, __fmul_rn(g1.y, O.z)));
    Oe.y = fmaf(g1.z, O.x, fmaf(g1.w, O.y, __fmul_rn(g2.x, O.z)));
    Oe.z = fmaf(g2.y, O.x, fmaf(g2.z, O.y, __fmul_rn(g2.w, O.z)));
    de.x = fmaf(g0.w, r.d.x, fmaf(g1.x, r.d.y, __fmul_rn(g1.y, r.d.z)));
    de.y = fmaf(g1.z, r.d.x, fmaf(g1.w, r.d.y, __fmul_rn(g2.x, r.d.z)));
    de.z = fmaf(g2.y, r.d.x, fmaf(g2.z, r.d.y, __fmul_rn(g2.w, r.d.z)));
    float a = dot3(de, de);
    float b = -dot3(Oe, de);
    float c = fmaf(Oe.x, Oe.x, fmaf(Oe.y, Oe.y, fmaf(Oe.z, Oe.z, -1.0f)));
    float inv_a = __fdividef(1.0f, a);
    float bia = __fmul_rn(b, inv_a);
    float3 P = make_float3(fmaf(bia, de.x, Oe.x), fmaf(bia, de.y, Oe.y), fmaf(bia, de.z, Oe.z));
    float disc = 1.0f - dot3(P, P);
    if (!(disc > 1e-7f)) return false;
    float sd = __fsqrt_rn(__fmul_rn(disc, a));
    float q = b + copysignf(sd, b);
    r1 = __fdiv_rn(c, q);
    r2 = __fmul_rn(q, inv_a);
    return true;
}

struct LeafTest {
    bool hit;
    float t_hit;     // max(tmin, root1, box entry) when hit
    float3 Oe, de;
};

__device__ __forceinline__ LeafTest test_gaussian(const MarchLaunch& L, const Ray& r, int j, bool valid, float tmin,
                                                  float tmax, Tally& tl, bool count) {
    LeafTest out;
    out.hit = false;
    out.t_hit = INFINITY;
    bool bh = false;
    float tnear = 0.f;
    if (valid) {
        float2 bx = __ldg(&L.h.bx[j]), by = __ldg(&L.h.by[j]), bz = __ldg(&L.h.bz[j]);
        bh = box_hit(r, bx, by, bz, tmin, tmax, tnear);
    }
    if (bh) {
        float4 g0 = __ldg(&L.g.g0[j]), g1 = __ldg(&L.g.g1[j]), g2 = __ldg(&L.g.g2[j]);
        float r1, r2;
        if (ellipsoid_interval(r, g0, g1, g2, out.Oe, out.de, r1, r2)) {
            float lo = fmaxf(tmin, r1), hi = fminf(tmax, r2);
            out.hit = lo <= hi;
            out.t_hit = fmaxf(lo, tnear);
        }
    }
    if (count) {
        tl.v[C_PRIM_TESTS] += __popc(__ballot_sync(kFull, valid));
        tl.v[C_ELL_TESTS] += __popc(__ballot_sync(kFull, bh));
    }
    return out;
}

// Any-hit search: calls leaf(LeafTest, j) once per group of 32 Gaussians whose
// parent box is hit, with all lanes converged; leaf returns false to stop.
template <bool COUNT, bool BRUTE, class LeafFn>
__device__ __forceinline__ void search_all(const MarchLaunch& L, const Ray& r, float tmin, float tmax, WarpShared& ws,
                                           int lane, Tally& tl, LeafFn&& leaf) {
    if (BRUTE) {
        for (int base = 0; base < L.g.n_pad; base += kFan) {
            int j = base + lane;
            LeafTest t = test_gaussian(L, r, j, j < L.g.n, tmin, tmax, tl, COUNT);
            if (!leaf(t, j)) return;
        }
        return;
    }
    const Hierarchy& h = L.h;
    const int top = h.num_levels - 1;
    int sp = 0;
    {
        bool bh = false;
        float tn;
        if (lane < h.count[top]) {
            int idx = h.offset[top] + lane;
            bh = box_hit(r, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), tmin, tmax, tn);
        }
        unsigned m = __ballot_sync(kFull, bh);
        if (bh) ws.stack[__popc(m & ((1u << lane) - 1u))] = ((uint32_t)top << 26) | (uint32_t)lane;
        sp = __popc(m);
        if (COUNT) tl.v[C_NODE_TESTS] += h.count[top];
        __syncwarp();
    }
    while (sp > 0) {
        uint32_t e = ws.stack[--sp];
        int level = (int)(e >> 26) - 1;          // level of the children
        int c = (int)(e & 0x3ffffffu) * kFan + lane;
        bool valid = c < h.count[level];
        if (level == 0) {
            LeafTest t = test_gaussian(L, r, c, valid, tmin, tmax, tl, COUNT);
            if (!leaf(t, c)) return;
        } else {
            bool bh = false;
            float tn;
            if (valid) {
                int idx = h.offset[level] + c;
                bh = box_hit(r, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), tmin, tmax, tn);
            }
            unsigned m = __ballot_sync(kFull, bh);
            int rank = __popc(m & ((1u << lane) - 1u));
            int n = __popc(m);
            if (sp + n > kStack) {               // never expected; drop the excess and report
                tl.v[C_STACK_OVF] += 1;
                n = kStack - sp;
            }
            if (bh && rank < n) ws.stack[sp + rank] = ((uint32_t)level << 26) | (uint32_t)c;
            sp += n;
            if (COUNT) tl.v[C_NODE_TESTS] += 32;
            __syncwarp();
        }
    }
}

// Closest-hit search over [tmin,tmax]: smallest t_hit, or +inf on a miss.
template <bool COUNT, bool BRUTE>
__device__ __forceinline__ float search_closest(const MarchLaunch& L, const Ray& r, float tmin, float tmax,
                                                WarpShared& ws, int lane, Tally& tl) {
    float best = INFINITY;
    if (COUNT) tl.v[C_CLOSEST] += 1;
    if (!(tmin <= tmax)) return best;
    if (BRUTE) {
        for (int base = 0; base < L.g.n_pad; base += kFan) {
            int j = base + lane;
            LeafTest t = test_gaussian(L, r, j, j < L.g.n, tmin, tmax, tl, COUNT);
            best = fminf(best, warp_min_f(t.hit ? t.t_hit : INFINITY));
        }
        return best;
    }
    const Hierarchy& h = L.h;
    const int top = h.num_levels - 1;
    int sp = 0;
    // pushes the hit children so that the nearest one is popped first
    auto push = [&](bool bh, float tn, int level, int c) {
        unsigned key = bh ? __float_as_uint(tn) : 0xffffffffu;      // tn >= tmin >= 0: order-preserving
        unsigned mn = __reduce_min_sync(kFull, key);
        unsigned near_mask = __ballot_sync(kFull, bh && key == mn);
        int near_lane = __ffs(near_mask) - 1;
        bool other = bh && lane != near_lane;
        unsigned m = __ballot_sync(kFull, other);
        int n = __popc(m), total = n + (near_lane >= 0 ? 1 : 0);
        if (sp + total > kStack) { tl.v[C_STACK_OVF] += 1; return; }
        if (other) {
            int s = sp + __popc(m & ((1u << lane) - 1u));
            ws.stack[s] = ((uint32_t)level << 26) | (uint32_t)c;
            ws.stack_t[s] = tn;
        }
        if (lane == near_lane) {
            ws.stack[sp + n] = ((uint32_t)level << 26) | (uint32_t)c;
            ws.stack_t[sp + n] = tn;
        }
        sp += total;
        __syncwarp();
    };
    {
        bool bh = false;
        float tn = 0.f;
        if (lane < h.count[top]) {
            int idx = h.offset[top] + lane;
            bh = box_hit(r, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), tmin, tmax, tn);
        }
        if (COUNT) tl.v[C_NODE_TESTS] += h.count[top];
        push(bh, tn, top, lane);
    }
    while (sp > 0) {
        --sp;
        uint32_t e = ws.stack[sp];
        float te = ws.stack_t[sp];
        if (te > best) continue;                 // nothing below this node can start earlier
        int level = (int)(e >> 26) - 1;
        int c = (int)(e & 0x3ffffffu) * kFan + lane;
        bool valid = c < h.count[level];
        if (level == 0) {
            LeafTest t = test_gaussian(L, r, c, valid, tmin, fminf(tmax, best), tl, COUNT);
            best = fminf(best, warp_min_f(t.hit ? t.t_hit : INFINITY));
            if (best <= tmin) return best;       // cannot improve on the interval start
        } else {
            bool bh = false;
            float tn = 0.f;
            if (valid) {
                int idx = h.offset[level] + c;
                bh = box_hit(r, __ldg(&h.bx[idx]), __ldg(&h.by[idx]), __ldg(&h.bz[idx]), tmin, fminf(tmax, best), tn);
            }
            if (COUNT) tl.v[C_NODE_TESTS] += 32;
            push(bh, tn, level, c);
        }
    }
    return best;
}

// ---------------------------------------------------------------- per-ray state machine shared by both passes
struct SlabPlan {
    float dt, slab, tmin, tmax;
    bool traced;
};

// cuda_train/forward/gaussians_aabb.cu:267-280
__device__ __forceinline__ SlabPlan plan_slab(const rgx_march& m, float tbuffer, float T, float tenter, float texit) {
    SlabPlan p;
    p.dt = m.dt_step;
    if (m.dynamic_sampling) {
        float dt_dist = fmaxf(__fdiv_rn(tbuffer, 1024.0f), m.dt_step);
        p.dt = fminf(__fmul_rn(dt_dist, rcbrtf(T)), __fmul_rn(4.0f, m.dt_step));
    }
    p.slab = __fmul_rn(p.dt, (float)kSlab);
    p.tmin = fmaxf(tenter, tbuffer);
    p.tmax = fminf(texit, __fadd_rn(tbuffer, p.slab));
    p.traced = p.tmax > tenter;
    return p;
}

// Scene-box clip, cuda_train/forward/gaussians_aabb.cu:212-224.
__device__ __forceinline__ void clip_scene(const SceneBox& b, const Ray& r, float& tenter, float& texit) {
    float t0x = __fmul_rn(b.lo[0] - r.o.x, r.inv.x), t1x = __fmul_rn(b.hi[0] - r.o.x, r.inv.x);
    float t0y = __fmul_rn(b.lo[1] - r.o.y, r.inv.y), t1y = __fmul_rn(b.hi[1] - r.o.y, r.inv.y);
    float t0z = __fmul_rn(b.lo[2] - r.o.z, r.inv.z), t1z = __fmul_rn(b.hi[2] - r.o.z, r.inv.z);
    tenter = fmaxf(0.0f, fmaxf(fminf(t0x, t1x), fmaxf(fminf(t0y, t1y), fminf(t0z, t1z))));
    texit = fminf(fmaxf(t0x, t1x), fminf(fmaxf(t0y, t1y), fmaxf(t0z, t1z)));
}

// Evaluate `count` staged Gaussians at this lane's sample: sums of sigma*g and of
// (payload)*g, payload being rgb*sigma in the forward (cuda_train/forward/gaussians_aabb.cu:166-178).
template <bool COUNT>
__device__ __forceinline__ void eval_forward(const WarpShared& ws, int count, float tau, float& s, float& cr,
                                             float& cg, float& cb, Tally& tl) {
#pragma unroll 2
    for (int j = 0; j < count; ++j) {
        float4 A = ws.recA[j], B = ws.recB[j], C = ws.recC[j];
        float yx = fmaf(tau, B.x, A.x), yy = fmaf(tau, B.y, A.y), yz = fmaf(tau, B.z, A.z);
        float q = fmaf(yx, yx, fmaf(yy, yy, __fmul_rn(yz, yz)));
        bool in = q < 1.0f;
        float e = in ? ex2_approx(__fmul_rn(-A.w, q)) : 0.0f;
        s = fmaf(B.w, e, s);
        cr = fmaf(C.x, e, cr);
        cg = fmaf(C.y, e, cg);
        cb = fmaf(C.z, e, cb);
        if (COUNT) tl.v[C_PAIRS] += __popc(__ballot_sync(kFull, in));
    }
}

__device__ __forceinline__ void flush_tally(const MarchLaunch& L, const Tally& tl, int lane) {
    if (L.counters && lane < 12 && tl.v[lane]) atomicAdd(&L.counters->v[lane], tl.v[lane]);
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
    return x;
}

// ---------------------------------------------------------------- forward
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
    for (int i = 0; i < 12; ++i) tl.v[i] = 0;

    for (int k = 0; k < kTile; ++k) {
        const int py = L.m.row_begin + tile_y * kTile + k;
        if (py >= L.m.row_end) break;
        const int ray_id = py * W + px;
        Ray r;
        make_ray(L.cam, px, py, r);
        float tenter, texit;
        clip_scene(box, r, tenter, texit);
        float T = 1.0f, Cr = 0.f, Cg = 0.f, Cb = 0.f, depth = 0.f;
        if (COUNT) tl.v[C_RAYS] += 1;

        float first = L.g.n > 0 ? search_closest<COUNT, BRUTE>(L, r, tenter, texit, ws, lane, tl) : INFINITY;
        if (first < INFINITY && first < texit) {                                  // :249-260
            tenter = first;
            float tbuffer = tenter;
            int slab_index = 0;
            while (tbuffer < texit && T > eps && slab_index < kMaxSlabs) {        // :266
                SlabPlan p = plan_slab(L.m, tbuffer, T, tenter, texit);
                if (COUNT) tl.v[C_SLABS] += 1;
                ++slab_index;
                if (!p.traced) { tbuffer = __fadd_rn(tbuffer, p.slab); continue; }
                float s = 0.f, cr = 0.f, cg = 0.f, cb = 0.f;
                const float tau = __fmul_rn((float)lane + 0.5f, p.dt);            // offset from tbuffer
                int nstage = 0, nhit = 0;
                bool overflow = false;
                search_all<COUNT, BRUTE>(L, r, p.tmin, p.tmax, ws, lane, tl, [&](const LeafTest& t, int j) {
                    unsigned m = __ballot_sync(kFull, t.hit);
                    if (m == 0u) return true;
                    int rank = __popc(m & ((1u << lane) - 1u)), n = __popc(m);
                    bool take = t.hit;
                    if (nhit + n > L.m.max_prim_slice) {                           // :352-356
                        n = L.m.max_prim_slice - nhit;
                        take = take && rank < n;
                        overflow = true;
                    }
                    if (take) {
                        int slot = nstage + rank;
                        float4 c = __ldg(&L.g.rgba[j]);
                        ws.recA[slot] = make_float4(fmaf(tbuffer, t.de.x, t.Oe.x), fmaf(tbuffer, t.de.y, t.Oe.y),
                                                    fmaf(tbuffer, t.de.z, t.Oe.z), __ldg(&L.g.hk[j]));
                        ws.recB[slot] = make_float4(t.de.x, t.de.y, t.de.z, c.w);
                        ws.recC[slot] = make_float4(c.x, c.y, c.z, 0.f);
                    }
                    if (COUNT) {
                        unsigned long long hsh = take ? mix64(((unsigned long long)ray_id << 40) ^
                                                              ((unsigned long long)slab_index << 24) ^
                                                              (unsigned long long)__ldg(&L.g.perm[j])) : 0ull;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) hsh += __shfl_xor_sync(kFull, hsh, o);
                        tl.v[C_HASH] += hsh;
                    }
                    nstage += n;
                    nhit += n;
                    __syncwarp();
                    if (nstage > kStage - kFan) {
                        eval_forward<COUNT>(ws, nstage, tau, s, cr, cg, cb, tl);
                        nstage = 0;
                        __syncwarp();
                    }
                    return !overflow;
                });
                if (nstage > 0) {
                    eval_forward<COUNT>(ws, nstage, tau, s, cr, cg, cb, tl);
                    __syncwarp();
                }
                if (COUNT) { tl.v[C_HITS] += nhit; tl.v[C_OVF] += overflow ? 1 : 0; }
                if (nhit == 0) {                                                  // :297-319
                    tbuffer = __fadd_rn(tbuffer, p.slab);
                    float nxt = search_closest<COUNT, BRUTE>(L, r, tbuffer, texit, ws, lane, tl);
                    if (!(nxt < INFINITY)) break;
                    tbuffer = nxt;
                    continue;
                }
                if (COUNT) tl.v[C_SLABS_HIT] += 1;
                // compositing, :190-201: lanes are samples; T before sample s is a prefix product
                float x = __fmul_rn(s, p.dt);
                float incl = warp_scan(x, lane);
                float excl = __fadd_rn(incl, -x);
                float w = exp_neg(x);
                float Ts = __fmul_rn(T, exp_neg(excl));
                float T16 = __shfl_sync(kFull, Ts, kChunk);
                bool live = lane < kChunk || T16 > eps;
                float one_m_w = 1.0f - w;
                float f = live ? __fmul_rn(Ts, __fmul_rn(p.dt, __fdividef(one_m_w, fmaxf(x, 1e-6f)))) : 0.f;
                Cr = __fadd_rn(Cr, warp_sum(__fmul_rn(f, cr)));
                Cg = __fadd_rn(Cg, warp_sum(__fmul_rn(f, cg)));
                Cb = __fadd_rn(Cb, warp_sum(__fmul_rn(f, cb)));
                if (L.depth) {
                    float ts = __fadd_rn(tbuffer, tau);
                    depth = __fadd_rn(depth, warp_sum(live ? __fmul_rn(__fmul_rn(Ts, one_m_w), ts) : 0.f));
                }
                float T32 = __fmul_rn(T, exp_neg(__shfl_sync(kFull, incl, 31)));
                T = (T16 > eps) ? T32 : T16;
                tbuffer = __fadd_rn(tbuffer, p.slab);                             // :324
            }
        }
        if (lane == 0) {                                                           // :326-339
            L.rgb[3 * (size_t)ray_id] = fmaf(T, bg, Cr);
            L.rgb[3 * (size_t)ray_id + 1] = fmaf(T, bg, Cg);
            L.rgb[3 * (size_t)ray_id + 2] = fmaf(T, bg, Cb);
            if (L.alpha) L.alpha[ray_id] = 1.0f - T;
            if (L.depth) L.depth[ray_id] = depth;
        }
    }
    if (COUNT) flush_tally(L, tl, lane);
}

// ---------------------------------------------------------------- backward
__device__ __forceinline__ void red_add_v4(float4* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

// Pass 2 over `count` staged Gaussians: each lane forms its sample's share of the
// four per-Gaussian sums, the warp adds them up, and lane j keeps the totals of
// staged Gaussian j.
//   recA = (y_c.xyz, hk)  recB = (de.xyz, tbuffer - t_c)  recC = (chat_i, -, -, -)
__device__ __forceinline__ void eval_backward(const WarpShared& ws, int count, float tau, float beta, float gamma,
                                              int lane, float& o_sb, float& o_n0, float& o_n1, float& o_n2) {
    for (int j = 0; j < count; ++j) {
        float4 A = ws.recA[j], B = ws.recB[j], C = ws.recC[j];
        float tc = __fadd_rn(tau, B.w);
        float yx = fmaf(tc, B.x, A.x), yy = fmaf(tc, B.y, A.y), yz = fmaf(tc, B.z, A.z);
        float q = fmaf(yx, yx, fmaf(yy, yy, __fmul_rn(yz, yz)));
        float e = q < 1.0f ? ex2_approx(__fmul_rn(-A.w, q)) : 0.0f;
        float ga = __fmul_rn(e, fmaf(C.x, beta, gamma));      // g * (alpha + beta*(chat_i - chat_s))
        float sb = warp_sum(__fmul_rn(e, beta));
        float n0 = warp_sum(ga);
        float g1 = __fmul_rn(ga, tc);
        float n1 = warp_sum(g1);
        float n2 = warp_sum(__fmul_rn(g1, tc));
        if (lane == j) { o_sb = sb; o_n0 = n0; o_n1 = n1; o_n2 = n2; }
    }
}

template <bool COUNT, bool BRUTE>
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
    for (int i = 0; i < 12; ++i) tl.v[i] = 0;

    for (int k = 0; k < kTile; ++k) {
        const int py = L.m.row_begin + tile_y * kTile + k;
        if (py >= L.m.row_end) break;
        const int ray_id = py * W + px;
        Ray r;
        make_ray(L.cam, px, py, r);
        float tenter, texit;
        clip_scene(box, r, tenter, texit);
        float first = L.g.n > 0 ? search_closest<COUNT, BRUTE>(L, r, tenter, texit, ws, lane, tl) : INFINITY;
        if (!(first < INFINITY && first < texit)) continue;                       // backward .cu:249-254
        tenter = first;
        const float3 dl = make_float3(L.dl_drgb[3 * (size_t)ray_id], L.dl_drgb[3 * (size_t)ray_id + 1],
                                      L.dl_drgb[3 * (size_t)ray_id + 2]);
        float D = fmaf(dl.x, L.rgb_in[3 * (size_t)ray_id],
                       fmaf(dl.y, L.rgb_in[3 * (size_t)ray_id + 1], dl.z * L.rgb_in[3 * (size_t)ray_id + 2]));
        float T = 1.0f;
        float tbuffer = tenter;
        int slab_index = 0;
        while (tbuffer < texit && T > eps && slab_index < kMaxSlabs) {
            SlabPlan p = plan_slab(L.m, tbuffer, T, tenter, texit);
            ++slab_index;
            if (!p.traced) { tbuffer = __fadd_rn(tbuffer, p.slab); continue; }
            const float tau = __fmul_rn((float)lane + 0.5f, p.dt);
            // ---- pass 1: per-sample sigma and delta.colour sums, same arithmetic as the forward
            float s = 0.f, dc = 0.f, u0 = 0.f, u1 = 0.f;
            int nstage = 0, nhit = 0;
            bool overflow = false;
            search_all<false, BRUTE>(L, r, p.tmin, p.tmax, ws, lane, tl, [&](const LeafTest& t, int j) {
                unsigned m = __ballot_sync(kFull, t.hit);
                if (m == 0u) return true;
                int rank = __popc(m & ((1u << lane) - 1u)), n = __popc(m);
                bool take = t.hit;
                if (nhit + n > L.m.max_prim_slice) {
                    n = L.m.max_prim_slice - nhit;
                    take = take && rank < n;
                    overflow = true;
                }
                if (take) {
                    int slot = nstage + rank;
                    float4 c = __ldg(&L.g.rgba[j]);
                    ws.recA[slot] = make_float4(fmaf(tbuffer, t.de.x, t.Oe.x), fmaf(tbuffer, t.de.y, t.Oe.y),
                                                fmaf(tbuffer, t.de.z, t.Oe.z), __ldg(&L.g.hk[j]));
                    ws.recB[slot] = make_float4(t.de.x, t.de.y, t.de.z, c.w);
                    ws.recC[slot] = make_float4(fmaf(dl.x, c.x, fmaf(dl.y, c.y, dl.z * c.z)), 0.f, 0.f, 0.f);
                }
                nstage += n;
                nhit += n;
                __syncwarp();
                if (nstage > kStage - kFan) {
                    eval_forward<false>(ws, nstage, tau, s, dc, u0, u1, tl);
                    nstage = 0;
                    __syncwarp();
                }
                return !overflow;
            });
            if (nstage > 0) {
                eval_forward<false>(ws, nstage, tau, s, dc, u0, u1, tl);
                __syncwarp();
            }
            if (nhit == 0) {
                tbuffer = __fadd_rn(tbuffer, p.slab);
                float nxt = search_closest<false, BRUTE>(L, r, tbuffer, texit, ws, lane, tl);
                if (!(nxt < INFINITY)) break;
                tbuffer = nxt;
                continue;
            }
            // ---- per-sample terms, backward .cu:330-352
            float x = __fmul_rn(s, p.dt);
            float incl = warp_scan(x, lane);
            float excl = __fadd_rn(incl, -x);
            float w = exp_neg(x);
            float Ts = __fmul_rn(T, exp_neg(excl));
            float T16 = __shfl_sync(kFull, Ts, kChunk);
            bool live = lane < kChunk || T16 > eps;                               // backward .cu:398
            float inv_s = s > 0.f ? __fdividef(1.0f, s) : 0.f;
            float chat = __fmul_rn(dc, inv_s);
            float one_m_w = 1.0f - w;
            float step = __fmul_rn(__fmul_rn(Ts, one_m_w), chat);                 // T_s (1-w_s) chat_s
            float sincl = warp_scan(step, lane);
            float Ds = __fadd_rn(D, -__fadd_rn(sincl, -step));
            float beta = live ? __fmul_rn(__fmul_rn(Ts, one_m_w), inv_s) : 0.f;
            float alpha = __fmul_rn(fmaf(Ts, chat, -Ds), p.dt);
            float gamma = live ? fmaf(-beta, chat, alpha) : 0.f;
            // ---- pass 2: same search again; gradients of every hit Gaussian
            int nhit2 = 0;
            nstage = 0;
            auto drain = [&]() {
                float sb = 0.f, n0 = 0.f, n1 = 0.f, n2 = 0.f;
                eval_backward(ws, nstage, tau, beta, gamma, lane, sb, n0, n1, n2);
                if (lane < nstage) {
                    const int j = prim_of[warp][lane];
                    const float4 A = ws.recA[lane], B = ws.recB[lane];
                    const float4 sd = __ldg(&L.g.sdens[j]);
                    const float4 qq = __ldg(&L.g.quat[j]);
                    const float4 g0 = __ldg(&L.g.g0[j]);
                    const float sigma = sd.w;
                    const float kk = __fsqrt_rn(__fmul_rn(2.0f * 0.6931471805599453f, A.w));    // k = sqrt(2 ln(sigma/sigma_t))
                    const float m0 = sigma * n0, m1 = sigma * n1, m2 = sigma * n2;
                    const float tc = __fadd_rn(tbuffer, -B.w);                    // reference point t_c
                    const float3 yc = make_float3(A.x, A.y, A.z), de = make_float3(B.x, B.y, B.z);
                    const float3 xc = make_float3(fmaf(tc, r.d.x, r.o.x - g0.x), fmaf(tc, r.d.y, r.o.y - g0.y),
                                                  fmaf(tc, r.d.z, r.o.z - g0.z));
                    const float inv_sc[3] = {1.0f / sd.x, 1.0f / sd.y, 1.0f / sd.z};
                    const float ycv[3] = {yc.x, yc.y, yc.z}, dev[3] = {de.x, de.y, de.z};
                    float3 U, V, Wc;
                    quat_to_columns(qq, U, V, Wc);
                    const float3 cols[3] = {U, V, Wc};
                    float dscale[3];
                    float3 dpos = make_float3(0.f, 0.f, 0.f);
                    float3 dcol[3];
                    const float k2 = kk * kk;
#pragma unroll
                    for (int a = 0; a < 3; ++a) {
                        // sum_s omega y_a^2 / s_a,  y = k (y_c + tc' de)
                        dscale[a] = k2 * (m0 * ycv[a] * ycv[a] + 2.0f * m1 * ycv[a] * dev[a] + m2 * dev[a] * dev[a]) *
                                    inv_sc[a];
                        const float coef = kk * (m0 * ycv[a] + m1 * dev[a]) * inv_sc[a];
                        dpos = dpos + cols[a] * coef;
                        // -(1/s_a) sum_s omega y_a (x_c + tc' d)
                        const float cx = kk * (m0 * ycv[a]) + kk * (m1 * dev[a]);
                        const float cd = kk * (m1 * ycv[a]) + kk * (m2 * dev[a]);
                        dcol[a] = (xc * cx + r.d * cd) * (-inv_sc[a]);
                    }
                    const float4 dq = quat_grad_from_columns(qq, dcol[0], dcol[1], dcol[2]);
                    const float cs = sigma * sb;
                    float4* row = L.grad_rows + 4 * (size_t)j;
                    red_add_v4(row, dpos.x, dpos.y, dpos.z, dscale[0]);
                    red_add_v4(row + 1, dscale[1], dscale[2], dq.x, dq.y);
                    red_add_v4(row + 2, dq.z, dq.w, n0, dl.x * cs);
                    red_add_v4(row + 3, dl.y * cs, dl.z * cs, 0.f, 0.f);
                }
                nstage = 0;
                __syncwarp();
            };
            search_all<false, BRUTE>(L, r, p.tmin, p.tmax, ws, lane, tl, [&](const LeafTest& t, int j) {
                unsigned m = __ballot_sync(kFull, t.hit);
                if (m == 0u) return true;
                int rank = __popc(m & ((1u << lane) - 1u)), n = __popc(m);
                bool take = t.hit;
                bool stop = false;
                if (nhit2 + n > L.m.max_prim_slice) {
                    n = L.m.max_prim_slice - nhit2;
                    take = take && rank < n;
                    stop = true;
                }
                if (nstage + n > kFan) drain();      // keep one staged Gaussian per lane
                if (take) {
                    int slot = nstage + rank;
                    float4 c = __ldg(&L.g.rgba[j]);
                    // reference point: closest approach clamped to the slab, so that moments stay small
                    float a = dot3(t.de, t.de);
                    float tca = __fdividef(-dot3(t.Oe, t.de), a);
                    tca = fminf(fmaxf(tca, tbuffer), __fadd_rn(tbuffer, p.slab));
                    ws.recA[slot] = make_float4(fmaf(tca, t.de.x, t.Oe.x), fmaf(tca, t.de.y, t.Oe.y),
                                                fmaf(tca, t.de.z, t.Oe.z), __ldg(&L.g.hk[j]));
                    ws.recB[slot] = make_float4(t.de.x, t.de.y, t.de.z, __fadd_rn(tbuffer, -tca));
                    float ci = __fdividef(fmaf(dl.x, c.x, fmaf(dl.y, c.y, dl.z * c.z)), c.w);
                    ws.recC[slot] = make_float4(ci, 0.f, 0.f, 0.f);
                    prim_of[warp][slot] = j;
                }
                nstage += n;
                nhit2 += n;
                __syncwarp();
                return !stop;
            });
            if (nstage > 0) drain();
            // ---- advance the ray state exactly as the forward does
            float T32 = __fmul_rn(T, exp_neg(__shfl_sync(kFull, incl, 31)));
            D = __fadd_rn(D, -__shfl_sync(kFull, sincl, 31));
            T = (T16 > eps) ? T32 : T16;
            tbuffer = __fadd_rn(tbuffer, p.slab);
        }
    }
    if (COUNT) flush_tally(L, tl, lane);
}

}  // namespace

static int grid_for(const MarchLaunch& m) {
    int rows = m.m.row_end - m.m.row_begin;
    if (rows <= 0 || m.cam.width <= 0) return 0;
    return ((m.cam.width + kTile - 1) / kTile) * ((rows + kTile - 1) / kTile);
}

cudaError_t launch_march_forward(const MarchLaunch& m, cudaStream_t s) {
    int grid = grid_for(m);
    if (grid == 0) return cudaSuccess;
    bool count = (m.m.flags & RGX_FLAG_COUNT_WORK) != 0, brute = (m.m.flags & RGX_FLAG_BRUTE_FORCE) != 0;
    if (count && brute) march_forward_kernel<true, true><<<grid, kWarps * 32, 0, s>>>(m);
    else if (count) march_forward_kernel<true, false><<<grid, kWarps * 32, 0, s>>>(m);
    else if (brute) march_forward_kernel<false, true><<<grid, kWarps * 32, 0, s>>>(m);
    else march_forward_kernel<false, false><<<grid, kWarps * 32, 0, s>>>(m);
    return cudaGetLastError();
}

cudaError_t launch_march_backward(const MarchLaunch& m, cudaStream_t s) {
    int grid = grid_for(m);
    if (grid == 0) return cudaSuccess;
    bool brute = (m.m.flags & RGX_FLAG_BRUTE_FORCE) != 0;
    if (brute) march_backward_kernel<false, true><<<grid, kWarps * 32, 0, s>>>(m);
    else march_backward_kernel<false, false><<<grid, kWarps * 32, 0, s>>>(m);
    return cudaGetLastError();
}

}  // namespace rgx
