// Device helpers shared by the march kernels: ray set-up, ray/box and
// ray/ellipsoid tests, enumeration of the Gaussians of a query by exhaustive loop
// or per-ray hierarchy search (the tile-list enumeration is in march_lists.cu),
// the slab schedule, the per-sample evaluation and the gradient of a hit.
#pragma once
#include "rgx_internal.cuh"
#include "device_math.cuh"

namespace rgx {

namespace {

constexpr int kWarps = 8;
constexpr int kStack = 192;
constexpr int kStage = 64;
constexpr unsigned kFull = 0xffffffffu;
constexpr int kTile = 8;   // per-ray variant (march.cu): a CTA marches 8x8 pixels, warp w takes column w
// Unrolling of the evaluation loop over staged hits (recording forward of the 3 M-Gaussian view: 1: 13.1 ms,
// 2: 11.9, 3: 11.9, 4: 11.8, 8: 11.8 -- but slabs with a handful of hits then run in the remainder loop).
#ifndef RGX_EVAL_UNROLL
#define RGX_EVAL_UNROLL 4
#endif
constexpr int kEvalUnroll = RGX_EVAL_UNROLL;
constexpr int kMaxSlabs = 1 << 22;   // hard bound on slab iterations per ray
#ifndef RGX_PACKED_FMA
#define RGX_PACKED_FMA 1
#endif

struct WarpStage {      // staged hit records of one warp
    float4 recA[kStage];
    float4 recB[kStage];
    float4 recC[kStage];
};
struct WarpShared : WarpStage {   // plus the search stack of the per-ray variant
    uint32_t stack[kStack];
    float stack_t[kStack];
};

struct Ray {
    float3 o, d, inv;
};

struct Tally {   // per-warp work counters (uniform across lanes)
    unsigned long long v[C_NUM];
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

// Ray origin and direction in the Gaussian's whitened frame (M = S^-1 R^T / k in g0..g2).
__device__ __forceinline__ void whiten_ray(const Ray& r, float4 g0, float4 g1, float4 g2, float3& Oe, float3& de) {
    float3 O = make_float3(r.o.x - g0.x, r.o.y - g0.y, r.o.z - g0.z);
    Oe.x = fmaf(g0.w, O.x, fmaf(g1.x, O.y, __fmul_rn(g1.y, O.z)));
    Oe.y = fmaf(g1.z, O.x, fmaf(g1.w, O.y, __fmul_rn(g2.x, O.z)));
    Oe.z = fmaf(g2.y, O.x, fmaf(g2.z, O.y, __fmul_rn(g2.w, O.z)));
    de.x = fmaf(g0.w, r.d.x, fmaf(g1.x, r.d.y, __fmul_rn(g1.y, r.d.z)));
    de.y = fmaf(g1.z, r.d.x, fmaf(g1.w, r.d.y, __fmul_rn(g2.x, r.d.z)));
    de.z = fmaf(g2.y, r.d.x, fmaf(g2.z, r.d.y, __fmul_rn(g2.w, r.d.z)));
}

// Interval of the ray inside the truncation ellipsoid
// (square root and the division for the first root are the approximate instructions, good to 2 ulp: the roots
// only decide whether and where the interval meets a slab; forward 10.2 -> 10.0 ms)
// (cuda_train/forward/gaussians_aabb.cu:43-91 with M = S^-1 R^T / k folded into g0..g2).
__device__ __forceinline__ bool ellipsoid_interval(const Ray& r, float4 g0, float4 g1, float4 g2, float3& Oe,
                                                   float3& de, float& r1, float& r2) {
    whiten_ray(r, g0, g1, g2, Oe, de);
    float a = dot3(de, de);
    float b = -dot3(Oe, de);
    float c = fmaf(Oe.x, Oe.x, fmaf(Oe.y, Oe.y, fmaf(Oe.z, Oe.z, -1.0f)));
    float inv_a = __fdividef(1.0f, a);
    float bia = __fmul_rn(b, inv_a);
    float3 P = make_float3(fmaf(bia, de.x, Oe.x), fmaf(bia, de.y, Oe.y), fmaf(bia, de.z, Oe.z));
    float disc = 1.0f - dot3(P, P);
    if (!(disc > 1e-7f)) return false;
    float sd = sqrt_approx(__fmul_rn(disc, a));
    float q = b + copysignf(sd, b);
    r1 = __fdividef(c, q);
    r2 = __fmul_rn(q, inv_a);
    return true;
}

struct LeafTest {
    bool hit;
    float t_hit;     // max(tmin, root1) when hit
    float3 Oe, de;
};

// The per-ray test that decides a hit: the reference's interval test on the truncation ellipsoid, nothing else
// (what its intersection program reports; its boxes only guide the traversal).  The Gaussian's box contains the
// ellipsoid with a margin well above the rounding of either test (build.cu), so testing it first (use_box)
// rejects no hit: the searches that come through boxes anyway keep it as a cheap first test, the march over
// tile lists, whose candidates pass it 94 times in 100, goes straight to the ellipsoid.
__device__ __forceinline__ LeafTest test_gaussian(const MarchLaunch& L, const Ray& r, int j, bool valid, float tmin,
                                                  float tmax, Tally& tl, bool count, bool use_box = true) {
    LeafTest out;
    out.hit = false;
    out.t_hit = INFINITY;
    bool bh = valid;
    if (use_box && valid) {
        float tnear;
        float2 bx = __ldg(&L.h.bx[j]), by = __ldg(&L.h.by[j]), bz = __ldg(&L.h.bz[j]);
        bh = box_hit(r, bx, by, bz, tmin, tmax, tnear);
    }
    if (bh) {
        float4 g0 = __ldg(&L.g.g0[j]), g1 = __ldg(&L.g.g1[j]), g2 = __ldg(&L.g.g2[j]);
        float r1, r2;
        if (ellipsoid_interval(r, g0, g1, g2, out.Oe, out.de, r1, r2)) {
            float lo = fmaxf(tmin, r1), hi = fminf(tmax, r2);
            out.hit = lo <= hi;
            out.t_hit = lo;
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
        sp = __popc(m);
        // lowest index on top: groups are then visited in ascending (Morton) order, as in the exhaustive scan
        if (bh) ws.stack[sp - 1 - __popc(m & ((1u << lane) - 1u))] = ((uint32_t)top << 26) | (uint32_t)lane;
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
            if (bh && rank < n) ws.stack[sp + n - 1 - rank] = ((uint32_t)level << 26) | (uint32_t)c;
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
        float dt_dist = fmaxf(__fmul_rn(tbuffer, 0.0009765625f), m.dt_step);      // t / 1024: a power of two, the same bits as the division
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
// Along a ray the whitened squared distance is a parabola in the sample position, q(tau) = q_min +
// |de|^2 (tau - tau*)^2 about the closest approach tau* (a sum of two non-negative terms: no cancellation), so a
// staged record is (tau*, (1 - q_min)/|de|^2, -hk |de|^2, -hk q_min) and (payload, sigma): the truncation
// test q < 1 is d^2 < (1 - q_min)/|de|^2 and the exponent one fused multiply-add of d^2.
// The four sums advance with two packed fp32x2 fused multiply-adds per hit (sm_100's FFMA2: two IEEE fp32 FMAs in
// one instruction, same bits as two scalar ones): the loop is bound by instruction issue, not by the FMA pipe.
template <bool COUNT>
__device__ __forceinline__ void eval_forward(const WarpStage& ws, int count, float tau, float& s, float& cr,
                                             float& cg, float& cb, Tally& tl) {
#if RGX_PACKED_FMA
    float2 rg = make_float2(cr, cg), bs = make_float2(cb, s);
#pragma unroll kEvalUnroll
    for (int j = 0; j < count; ++j) {
        const float4 A = ws.recA[j], C = ws.recB[j];
        const float d = __fadd_rn(tau, -A.x);
        const float d2 = __fmul_rn(d, d);
        const bool in = d2 < A.y;
        const float e = in ? ex2_approx(fmaf(A.z, d2, A.w)) : 0.0f;
        const float2 ee = make_float2(e, e);
        rg = __ffma2_rn(make_float2(C.x, C.y), ee, rg);
        bs = __ffma2_rn(make_float2(C.z, C.w), ee, bs);
        if (COUNT) tl.v[C_PAIRS] += __popc(__ballot_sync(kFull, in));
    }
    cr = rg.x; cg = rg.y; cb = bs.x; s = bs.y;
#else
#pragma unroll kEvalUnroll
    for (int j = 0; j < count; ++j) {
        const float4 A = ws.recA[j], C = ws.recB[j];
        const float d = __fadd_rn(tau, -A.x);
        const float d2 = __fmul_rn(d, d);
        const bool in = d2 < A.y;
        const float e = in ? ex2_approx(fmaf(A.z, d2, A.w)) : 0.0f;
        s = fmaf(C.w, e, s);
        cr = fmaf(C.x, e, cr);
        cg = fmaf(C.y, e, cg);
        cb = fmaf(C.z, e, cb);
        if (COUNT) tl.v[C_PAIRS] += __popc(__ballot_sync(kFull, in));
    }
#endif
}

// The record of eval_forward for a hit with whitened ray origin Oe and direction de, sample positions counted
// from tbuffer; hk is the exponent scale of ex2 (response = ex2(-hk q)).
__device__ __forceinline__ float4 parabola_record(float3 Oe, float3 de, float tbuffer, float hk) {
    const float a = dot3(de, de);
    const float tstar = __fdiv_rn(-dot3(Oe, de), a);
    const float3 P = make_float3(fmaf(tstar, de.x, Oe.x), fmaf(tstar, de.y, Oe.y), fmaf(tstar, de.z, Oe.z));
    const float qmin = dot3(P, P);
    return make_float4(__fadd_rn(tstar, -tbuffer), __fdividef(1.0f - qmin, a), __fmul_rn(-hk, a), __fmul_rn(-hk, qmin));
}

__device__ __forceinline__ void flush_tally(const MarchLaunch& L, const Tally& tl, int lane) {
    if (L.counters && lane < C_NUM && tl.v[lane]) atomicAdd(&L.counters->v[lane], tl.v[lane]);
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
    return x;
}


__device__ __forceinline__ void red_add_v4(float4* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

// Sums eight per-lane values over the warp at once: on return every lane holds the
// warp total of v[(lane >> 2) & 7].  9 shuffles instead of 8 x 5.
__device__ __forceinline__ float reduce8(const float (&v)[8], int lane) {
    float a[4], b[2];
    bool up = (lane & 16) != 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        float recv = __shfl_xor_sync(kFull, up ? v[t] : v[t + 4], 16);
        a[t] = __fadd_rn(up ? v[t + 4] : v[t], recv);
    }
    up = (lane & 8) != 0;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        float recv = __shfl_xor_sync(kFull, up ? a[t] : a[t + 2], 8);
        b[t] = __fadd_rn(up ? a[t + 2] : a[t], recv);
    }
    up = (lane & 4) != 0;
    float recv = __shfl_xor_sync(kFull, up ? b[0] : b[1], 4);
    float c = __fadd_rn(up ? b[1] : b[0], recv);
    c = __fadd_rn(c, __shfl_xor_sync(kFull, c, 2));
    c = __fadd_rn(c, __shfl_xor_sync(kFull, c, 1));
    return c;
}

// Pass 2 over `count` (<= 32) staged Gaussians: each lane forms its sample's share of
// the four per-Gaussian sums, the warp adds them up eight Gaussians at a time, and
// lane j keeps the totals of staged Gaussian j.
//   recA = (y_c.xyz, hk)  recB = (de.xyz, tbuffer - t_c)  recC = (chat_i, -, -, -)
__device__ __forceinline__ void eval_backward(const WarpStage& ws, int count, float tau, float beta, float gamma,
                                              int lane, float& o_sb, float& o_n0, float& o_n1, float& o_n2) {
    for (int j0 = 0; j0 < count; j0 += 8) {
        float vb[8], v0[8], v1[8], v2[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int j = j0 + e;
            if (j < count) {
                float4 A = ws.recA[j], B = ws.recB[j], C = ws.recC[j];
                float tc = __fadd_rn(tau, B.w);
                float yx = fmaf(tc, B.x, A.x), yy = fmaf(tc, B.y, A.y), yz = fmaf(tc, B.z, A.z);
                float q = fmaf(yx, yx, fmaf(yy, yy, __fmul_rn(yz, yz)));
                float ex = q < 1.0f ? ex2_approx(__fmul_rn(-A.w, q)) : 0.0f;
                float ga = __fmul_rn(ex, fmaf(C.x, beta, gamma));      // g * (alpha + beta*(chat_i - chat_s))
                float g1 = __fmul_rn(ga, tc);
                vb[e] = __fmul_rn(ex, beta); v0[e] = ga; v1[e] = g1; v2[e] = __fmul_rn(g1, tc);
            } else {
                vb[e] = v0[e] = v1[e] = v2[e] = 0.f;
            }
        }
        const float rb = reduce8(vb, lane), r0 = reduce8(v0, lane), r1 = reduce8(v1, lane), r2 = reduce8(v2, lane);
        // the totals of staged Gaussian j0 + e sit in lanes 4e .. 4e+3; hand them to lane j0 + e
        const int src = 4 * ((lane - j0) & 7);
        const float tb = __shfl_sync(kFull, rb, src), t0 = __shfl_sync(kFull, r0, src), t1 = __shfl_sync(kFull, r1, src),
                    t2 = __shfl_sync(kFull, r2, src);
        if (lane >= j0 && lane < j0 + 8) { o_sb = tb; o_n0 = t0; o_n1 = t1; o_n2 = t2; }
    }
}

// ---------------------------------------------------------------- one slab, generic over how Gaussians are enumerated
//
// `enumerate(leaf)` must call leaf(LeafTest, j) for groups of up to 32 Gaussians in
// ascending sorted index j, all lanes converged, until leaf returns false.  The
// three enumerations (exhaustive, per-ray hierarchy search, candidate list) give
// the same hits in the same order, hence bit-identical sums.

// Per-sample sums of sigma*g (s) and payload*g (c0..c2); payload is rgb*sigma in
// the forward and (dl . rgb*sigma, 0, 0) in the backward.  Returns the hit count.
template <bool COUNT, bool BWD, class Enum>
__device__ __forceinline__ int slab_sums(const MarchLaunch& L, const rgx_march& m, float tbuffer, float tau,
                                         int ray_id, int slab_index, float3 dl, WarpStage& ws, int lane, Tally& tl,
                                         Enum&& enumerate, float& s, float& c0, float& c1, float& c2,
                                         bool& overflow, int* const* hit_list = nullptr, int hit_cap = 0) {
    int nstage = 0, nhit = 0;
    bool ovf = false;
    s = c0 = c1 = c2 = 0.f;
    enumerate([&](const LeafTest& t, int j) {
        unsigned mask = __ballot_sync(kFull, t.hit);
        if (mask == 0u) return true;
        const long long c_s = COUNT ? clock64() : 0;
        int rank = __popc(mask & ((1u << lane) - 1u)), n = __popc(mask);
        bool take = t.hit;
        if (nhit + n > m.max_prim_slice) {            // cuda_train/forward/gaussians_aabb.cu:352-356
            n = m.max_prim_slice - nhit;
            take = take && rank < n;
            ovf = true;
        }
        if (take) {
            int slot = nstage + rank;
            if (hit_list) {                      // remembered for the second pass; *hit_list may be null
                int* list = *hit_list;
                if (list && nhit + rank < hit_cap) list[nhit + rank] = j;
            }
            const float4 c = __ldg(&L.g.rgba[j]);       // (rgb sigma, sigma)
            ws.recA[slot] = parabola_record(t.Oe, t.de, tbuffer, __ldg(&L.g.hk[j]));
            ws.recB[slot] = BWD ? make_float4(fmaf(dl.x, c.x, fmaf(dl.y, c.y, __fmul_rn(dl.z, c.z))), 0.f, 0.f, c.w) : c;
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
        if (COUNT) tl.v[C_CYC_WINDOW] += clock64() - c_s;       // staging of the hits
        if (nstage > kStage - kFan) {
            long long c_a = COUNT ? clock64() : 0;
            eval_forward<COUNT>(ws, nstage, tau, s, c0, c1, c2, tl);
            nstage = 0;
            __syncwarp();
            if (COUNT) tl.v[C_CYC_EVAL] += clock64() - c_a;
        }
        return !ovf;
    });
    if (nstage > 0) {
        long long c_a = COUNT ? clock64() : 0;
        eval_forward<COUNT>(ws, nstage, tau, s, c0, c1, c2, tl);
        __syncwarp();
        if (COUNT) tl.v[C_CYC_EVAL] += clock64() - c_a;
    }
    overflow = ovf;
    return nhit;
}

// Transmittance bookkeeping of one slab (cuda_train/forward/gaussians_aabb.cu:190-201):
// lanes are samples, the transmittance before sample s is a prefix product, and the
// second chunk of 16 samples only counts if T is still above the threshold after the first.
struct SlabTrans {
    float x, w, Ts, incl, T16, T32;
    bool live;
};
__device__ __forceinline__ SlabTrans slab_transmittance(float s, float dt, float T, float eps, int lane) {
    SlabTrans o;
    o.x = __fmul_rn(s, dt);
    o.incl = warp_scan(o.x, lane);
    float excl = __fadd_rn(o.incl, -o.x);
    o.w = exp_neg(o.x);
    o.Ts = __fmul_rn(T, exp_neg(excl));
    o.T16 = __shfl_sync(kFull, o.Ts, kChunk);
    o.live = lane < kChunk || o.T16 > eps;
    o.T32 = __fmul_rn(T, exp_neg(__shfl_sync(kFull, o.incl, 31)));
    return o;
}
__device__ __forceinline__ float slab_exit_T(const SlabTrans& o, float eps) { return (o.T16 > eps) ? o.T32 : o.T16; }

struct RayColor {
    float T, Cr, Cg, Cb, depth;
};

__device__ __forceinline__ void composite_forward(const SlabPlan& p, float tbuffer, float tau, float eps, int lane,
                                                  float s, float cr, float cg, float cb, bool want_depth,
                                                  RayColor& st) {
    SlabTrans tr = slab_transmittance(s, p.dt, st.T, eps, lane);
    float one_m_w = 1.0f - tr.w;
    float f = tr.live ? __fmul_rn(tr.Ts, __fmul_rn(p.dt, __fdividef(one_m_w, fmaxf(tr.x, 1e-6f)))) : 0.f;
    st.Cr = __fadd_rn(st.Cr, warp_sum(__fmul_rn(f, cr)));
    st.Cg = __fadd_rn(st.Cg, warp_sum(__fmul_rn(f, cg)));
    st.Cb = __fadd_rn(st.Cb, warp_sum(__fmul_rn(f, cb)));
    if (want_depth) {
        float ts = __fadd_rn(tbuffer, tau);
        st.depth = __fadd_rn(st.depth, warp_sum(tr.live ? __fmul_rn(__fmul_rn(tr.Ts, one_m_w), ts) : 0.f));
    }
    st.T = slab_exit_T(tr, eps);
}

// The same with the ray's colour and depth kept in shared memory (x, y, z = colour, w = depth; lane 0 owns
// them): they are touched once per slab, and the registers are wanted elsewhere all the time.
__device__ __forceinline__ void composite_forward_shared(const SlabPlan& p, float tbuffer, float tau, float eps, int lane,
                                                         float s, float cr, float cg, float cb, bool want_depth,
                                                         float& T, float4* acc) {
    SlabTrans tr = slab_transmittance(s, p.dt, T, eps, lane);
    float one_m_w = 1.0f - tr.w;
    float f = tr.live ? __fmul_rn(tr.Ts, __fmul_rn(p.dt, __fdividef(one_m_w, fmaxf(tr.x, 1e-6f)))) : 0.f;
    const float sr = warp_sum(__fmul_rn(f, cr)), sg = warp_sum(__fmul_rn(f, cg)), sb = warp_sum(__fmul_rn(f, cb));
    float sd = 0.f;
    if (want_depth) {
        float ts = __fadd_rn(tbuffer, tau);
        sd = warp_sum(tr.live ? __fmul_rn(__fmul_rn(tr.Ts, one_m_w), ts) : 0.f);
    }
    if (lane == 0) {
        float4 a = *acc;
        *acc = make_float4(__fadd_rn(a.x, sr), __fadd_rn(a.y, sg), __fadd_rn(a.z, sb), __fadd_rn(a.w, sd));
    }
    T = slab_exit_T(tr, eps);
}

// 8-bit colour of the reference's viewer (cuda_gui/helpers.h:45-58): clamp to [0,1], times 256,
// truncate, at most 255; no gamma.
__device__ __forceinline__ unsigned char quantize8(float x) {
    x = fminf(fmaxf(x, 0.0f), 1.0f);
    return (unsigned char)min((unsigned int)__fmul_rn(x, 256.0f), 255u);
}

// What a ray leaves behind (cuda_train/forward/gaussians_aabb.cu:326-339; cuda_gui/gaussians_aabb.cu:330-342).
__device__ __forceinline__ void write_ray(const MarchLaunch& L, int ray_id, const RayColor& st, float bg) {
    const float r = fmaf(st.T, bg, st.Cr), g = fmaf(st.T, bg, st.Cg), b = fmaf(st.T, bg, st.Cb);
    if (L.rgb) { L.rgb[3 * (size_t)ray_id] = r; L.rgb[3 * (size_t)ray_id + 1] = g; L.rgb[3 * (size_t)ray_id + 2] = b; }
    if (L.frame) L.frame[ray_id] = make_uchar4(quantize8(r), quantize8(g), quantize8(b), 255u);
    if (L.alpha) L.alpha[ray_id] = 1.0f - st.T;
    if (L.depth) L.depth[ray_id] = st.depth;
}

// Per-sample terms of the backward (cuda_train/backward/gaussians_aabb.cu:330-352).
struct SlabBackTerms {
    float beta, gamma, d_total;
    SlabTrans tr;
};
__device__ __forceinline__ SlabBackTerms slab_back_terms(float s, float dc, float dt, float T, float D, float eps,
                                                         int lane) {
    SlabBackTerms o;
    o.tr = slab_transmittance(s, dt, T, eps, lane);
    float inv_s = s > 0.f ? __fdividef(1.0f, s) : 0.f;
    float chat = __fmul_rn(dc, inv_s);
    float one_m_w = 1.0f - o.tr.w;
    float step = __fmul_rn(__fmul_rn(o.tr.Ts, one_m_w), chat);                 // T_s (1-w_s) chat_s
    float sincl = warp_scan(step, lane);
    float Ds = __fadd_rn(D, -__fadd_rn(sincl, -step));
    o.beta = o.tr.live ? __fmul_rn(__fmul_rn(o.tr.Ts, one_m_w), inv_s) : 0.f;
    float alpha = __fmul_rn(fmaf(o.tr.Ts, chat, -Ds), dt);
    o.gamma = o.tr.live ? fmaf(-o.beta, chat, alpha) : 0.f;
    o.d_total = __shfl_sync(kFull, sincl, 31);
    return o;
}

// Gradient of one (ray, slab, Gaussian) triple from its four moment sums.  The
// sample-wise sums of cuda_train/backward/gaussians_aabb.cu:401-441 collapse because
// the whitened offset y = y_c + t' de is affine in the sample position: with the
// weights w_s (sigma times the sample's share of the loss gradient) everything the
// chain rule needs is the first moment mu = sum_s w_s y_s and the second moment
// Y = sum_s w_s y_s y_s^T, both in the Gaussian's whitened frame.  The march adds
// those up per Gaussian; the step to position, scale and quaternion gradients is
// taken once per Gaussian afterwards (finalize_kernel), not once per hit.
struct GaussGrad {
    float3 mu;
    float y00, y11, y22, y01, y02, y12;
    float dsigma;
    float drgb_scale;   // dL/drgb = dl * drgb_scale
};
// A = (y_c.xyz, -), B = (de.xyz, -): the whitened ray point at the reference parameter and the whitened direction
__device__ __forceinline__ GaussGrad expand_gradient(float sigma, float4 A, float4 B, float sb, float n0, float n1,
                                                     float n2) {
    const float m0 = __fmul_rn(sigma, n0), m1 = __fmul_rn(sigma, n1), m2 = __fmul_rn(sigma, n2);
    const float3 yc = make_float3(A.x, A.y, A.z), de = make_float3(B.x, B.y, B.z);
    const float3 U = make_float3(fmaf(m0, yc.x, __fmul_rn(m1, de.x)), fmaf(m0, yc.y, __fmul_rn(m1, de.y)),
                                 fmaf(m0, yc.z, __fmul_rn(m1, de.z)));
    const float3 V = make_float3(fmaf(m1, yc.x, __fmul_rn(m2, de.x)), fmaf(m1, yc.y, __fmul_rn(m2, de.y)),
                                 fmaf(m1, yc.z, __fmul_rn(m2, de.z)));
    GaussGrad g;
    g.mu = U;
    g.y00 = fmaf(yc.x, U.x, __fmul_rn(de.x, V.x));
    g.y11 = fmaf(yc.y, U.y, __fmul_rn(de.y, V.y));
    g.y22 = fmaf(yc.z, U.z, __fmul_rn(de.z, V.z));
    g.y01 = fmaf(yc.x, U.y, __fmul_rn(de.x, V.y));
    g.y02 = fmaf(yc.x, U.z, __fmul_rn(de.x, V.z));
    g.y12 = fmaf(yc.y, U.z, __fmul_rn(de.y, V.z));
    g.dsigma = n0;
    g.drgb_scale = __fmul_rn(sigma, sb);
    return g;
}

// Pass 2 of the backward for one slab: enumerate the same hits again and hand the
// gradient of every (slab, Gaussian) pair to emit(j, GaussGrad) on the owning lane.
template <class Enum, class Emit>
__device__ __forceinline__ void slab_gradients(const MarchLaunch& L, const rgx_march& m, const Ray& r,
                                               const SlabPlan& p, float tbuffer, float tau, float3 dl, float beta,
                                               float gamma, WarpStage& ws, int* prim_of, int lane,
                                               Enum&& enumerate, Emit&& emit) {
    int nstage = 0, nhit = 0;
    auto drain = [&]() {
        float sb = 0.f, n0 = 0.f, n1 = 0.f, n2 = 0.f;
        eval_backward(ws, nstage, tau, beta, gamma, lane, sb, n0, n1, n2);
        if (lane < nstage) {
            const int j = prim_of[lane];
            emit(j, expand_gradient(__ldg(&L.g.sdens[j]).w, ws.recA[lane], ws.recB[lane], sb, n0, n1, n2));
        }
        nstage = 0;
        __syncwarp();
    };
    enumerate([&](const LeafTest& t, int j) {
        unsigned mask = __ballot_sync(kFull, t.hit);
        if (mask == 0u) return true;
        int rank = __popc(mask & ((1u << lane) - 1u)), n = __popc(mask);
        bool take = t.hit;
        bool stop = false;
        if (nhit + n > m.max_prim_slice) {
            n = m.max_prim_slice - nhit;
            take = take && rank < n;
            stop = true;
        }
        if (nstage + n > kFan) drain();          // one staged Gaussian per lane
        if (take) {
            int slot = nstage + rank;
            float4 c = __ldg(&L.g.rgba[j]);
            // reference point: closest approach clamped to the slab, so that the moments stay small
            float a = dot3(t.de, t.de);
            float tca = __fdividef(-dot3(t.Oe, t.de), a);
            tca = fminf(fmaxf(tca, tbuffer), __fadd_rn(tbuffer, p.slab));
            ws.recA[slot] = make_float4(fmaf(tca, t.de.x, t.Oe.x), fmaf(tca, t.de.y, t.Oe.y),
                                        fmaf(tca, t.de.z, t.Oe.z), __ldg(&L.g.hk[j]));
            ws.recB[slot] = make_float4(t.de.x, t.de.y, t.de.z, __fadd_rn(tbuffer, -tca));
            float ci = __fdividef(fmaf(dl.x, c.x, fmaf(dl.y, c.y, __fmul_rn(dl.z, c.z))), c.w);
            ws.recC[slot] = make_float4(ci, 0.f, 0.f, 0.f);
            prim_of[slot] = j;
        }
        nstage += n;
        nhit += n;
        __syncwarp();
        return !stop;
    });
    if (nstage > 0) drain();
}

// Row layout of grad_rows, [copies, n_pad, 4] float4 per sorted slot:
//   (mu.xyz, Y00) (Y11, Y22, Y01, Y02) (Y12, dsigma, drgb.xy) (drgb.z, -, -, -)
// A Gaussian that fills the view is met by every ray, and additions to one address queue up in
// the L2; CTAs therefore spread over `copies` sets of rows, which finalize_kernel adds up.
// `spread`: what chooses the copy (the CTA's tile, so that the CTAs that share a tile -- and its Gaussians -- share rows).
__device__ __forceinline__ void emit_global(const MarchLaunch& L, float3 dl, int j, const GaussGrad& g, unsigned spread) {
    float4* row = L.grad_rows + 4 * ((size_t)(spread & (unsigned)(L.grad_copies - 1)) * (size_t)L.g.n_pad + (size_t)j);
    red_add_v4(row, g.mu.x, g.mu.y, g.mu.z, g.y00);
    red_add_v4(row + 1, g.y11, g.y22, g.y01, g.y02);
    red_add_v4(row + 2, g.y12, g.dsigma, __fmul_rn(dl.x, g.drgb_scale), __fmul_rn(dl.y, g.drgb_scale));
    atomicAdd(reinterpret_cast<float*>(row + 3), __fmul_rn(dl.z, g.drgb_scale));
}

}  // namespace

}  // namespace rgx
