// Acceleration-structure build: per-Gaussian boxes, scene box, Morton keys,
// radix sort, sorted per-Gaussian records and a bottom-up refit of a 32-ary
// hierarchy.  Runs once per parameter version.
//
// Takes the place of ellipsoids_bbox_from_quat + create_acceleration_structure of
// the reference (optix_raycasting/optix_utils.py:36-109,139-142), where the
// hierarchy itself is built inside the OptiX driver.
#include "rgx_internal.cuh"
#include "device_math.cuh"
#include <cub/device/device_radix_sort.cuh>

namespace rgx {

namespace {

__device__ __forceinline__ int float_to_ordered(float f) {
    int i = __float_as_int(f);
    return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_to_float(int i) {
    return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void init_bounds_kernel(int* bounds) {
    int t = threadIdx.x;
    if (t < 12) {
        bool is_lo = (t % 6) < 3;
        bounds[t] = float_to_ordered(is_lo ? INFINITY : -INFINITY);
    }
}

// One thread per Gaussian: scene box over every Gaussian's box (degenerate ones
// included, as the reference's min/max reductions do) and the box of the centres.
__global__ void __launch_bounds__(256) bounds_kernel(BuildLaunch b) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    float lo[3] = {INFINITY, INFINITY, INFINITY}, hi[3] = {-INFINITY, -INFINITY, -INFINITY};
    float clo[3] = {INFINITY, INFINITY, INFINITY}, chi[3] = {-INFINITY, -INFINITY, -INFINITY};
    if (i < b.sc.n) {
        float3 p = make_float3(b.sc.positions[3 * i], b.sc.positions[3 * i + 1], b.sc.positions[3 * i + 2]);
        float3 s = make_float3(b.sc.scales[3 * i], b.sc.scales[3 * i + 1], b.sc.scales[3 * i + 2]);
        float4 q = reinterpret_cast<const float4*>(b.sc.quaternions)[i];
        float3 blo, bhi;
        gaussian_aabb(p, s, q, b.sc.densities[i], b.sigma_threshold, blo, bhi);
        lo[0] = blo.x; lo[1] = blo.y; lo[2] = blo.z;
        hi[0] = bhi.x; hi[1] = bhi.y; hi[2] = bhi.z;
        if (isfinite(p.x) && isfinite(p.y) && isfinite(p.z)) {
            clo[0] = chi[0] = p.x; clo[1] = chi[1] = p.y; clo[2] = chi[2] = p.z;
        }
    }
    __shared__ float red[12][8];
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        float v0 = warp_min(lo[a]), v1 = warp_max(hi[a]), v2 = warp_min(clo[a]), v3 = warp_max(chi[a]);
        if (lane == 0) { red[a][warp] = v0; red[3 + a][warp] = v1; red[6 + a][warp] = v2; red[9 + a][warp] = v3; }
    }
    __syncthreads();
    if (threadIdx.x < 12) {
        int t = threadIdx.x;
        bool is_lo = (t % 6) < 3;
        float v = red[t][0];
        for (int w = 1; w < 8; ++w) v = is_lo ? fminf(v, red[t][w]) : fmaxf(v, red[t][w]);
        if (is_lo) atomicMin(&b.bounds[t], float_to_ordered(v));
        else atomicMax(&b.bounds[t], float_to_ordered(v));
    }
}

__device__ __forceinline__ uint64_t spread3(uint64_t x) {
    x &= 0x1fffffull;
    x = (x | x << 32) & 0x1f00000000ffffull;
    x = (x | x << 16) & 0x1f0000ff0000ffull;
    x = (x | x << 8) & 0x100f00f00f00f00full;
    x = (x | x << 4) & 0x10c30c30c30c30c3ull;
    x = (x | x << 2) & 0x1249249249249249ull;
    return x;
}

// Cell coordinates -> "transposed" Hilbert index (J. Skilling, "Programming the
// Hilbert curve", AIP Conf. Proc. 707, 2004): after the call, interleaving the bits
// of q[0], q[1], q[2] (q[0] most significant) gives the position along the curve.
// Unlike a Morton curve, a run of consecutive Hilbert indices is always a connected
// set of cells, so fixed-size groups of sorted Gaussians get tighter boxes.
__device__ __forceinline__ void hilbert_transpose(uint32_t* q, int bits) {
    const uint32_t top = 1u << (bits - 1);
    for (uint32_t Q = top; Q > 1; Q >>= 1) {
        const uint32_t P = Q - 1;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            if (q[i] & Q) q[0] ^= P;
            else { uint32_t t = (q[0] ^ q[i]) & P; q[0] ^= t; q[i] ^= t; }
        }
    }
    q[1] ^= q[0];
    q[2] ^= q[1];
    uint32_t t = 0;
    for (uint32_t Q = top; Q > 1; Q >>= 1)
        if (q[2] & Q) t ^= Q - 1;
    q[0] ^= t; q[1] ^= t; q[2] ^= t;
}

__global__ void __launch_bounds__(256) morton_kernel(BuildLaunch b) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) {
        for (int a = 0; a < 3; ++a) {
            b.box->lo[a] = ordered_to_float(b.bounds[a]);
            b.box->hi[a] = ordered_to_float(b.bounds[3 + a]);
        }
    }
    if (i >= b.sc.n) return;
    const float cells = (float)(1u << b.morton_bits);
    uint32_t q[3];
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        float lo = ordered_to_float(b.bounds[6 + a]), hi = ordered_to_float(b.bounds[9 + a]);
        float ext = hi - lo;
        float u = ext > 0.f ? (b.sc.positions[3 * i + a] - lo) / ext : 0.f;
        u = fminf(fmaxf(u * cells, 0.f), cells - 1.f);
        if (!(u == u)) u = 0.f;
        q[a] = (uint32_t)u;
    }
    uint64_t key;
    if (b.curve == RGX_CURVE_HILBERT) {
        hilbert_transpose(q, b.morton_bits);
        key = (spread3(q[0]) << 2) | (spread3(q[1]) << 1) | spread3(q[2]);
    } else {
        key = spread3(q[0]) | (spread3(q[1]) << 1) | (spread3(q[2]) << 2);
    }
    b.keys_in[i] = key;
    b.vals_in[i] = (uint32_t)i;
}

// One thread per sorted slot: whitening matrix, truncation constant, raw copies
// for the backward, and the level-0 box.
__global__ void __launch_bounds__(256) gather_kernel(BuildLaunch b) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= b.n_pad) return;
    const float nanv = __int_as_float(0x7fc00000);
    float4 g0 = make_float4(0.f, 0.f, 0.f, nanv), g1 = make_float4(nanv, nanv, nanv, nanv), g2 = g1;
    float4 qq = make_float4(1.f, 0.f, 0.f, 0.f), sd = make_float4(1.f, 1.f, 1.f, 0.f);
    float hk = 0.f;
    float3 lo = make_float3(FLT_MAX, FLT_MAX, FLT_MAX), hi = make_float3(-FLT_MAX, -FLT_MAX, -FLT_MAX);
    if (j < b.sc.n) {
        int i = (int)b.vals_out[j];
        float3 p = make_float3(b.sc.positions[3 * i], b.sc.positions[3 * i + 1], b.sc.positions[3 * i + 2]);
        float3 s = make_float3(b.sc.scales[3 * i], b.sc.scales[3 * i + 1], b.sc.scales[3 * i + 2]);
        float4 q = reinterpret_cast<const float4*>(b.sc.quaternions)[i];
        float dens = b.sc.densities[i];
        qq = q;
        sd = make_float4(s.x, s.y, s.z, dens);
        g0.x = p.x; g0.y = p.y; g0.z = p.z;
        float ratio = dens / b.sigma_threshold;
        float k2 = 2.0f * logf(ratio);                   // optix_utils.py:287
        if (dens > b.sigma_threshold && k2 > 0.f && isfinite(k2)) {
            float k = sqrtf(k2);
            float3 U, V, W;
            quat_to_columns(q, U, V, W);
            float ix = 1.0f / (s.x * k), iy = 1.0f / (s.y * k), iz = 1.0f / (s.z * k);
            g0.w = U.x * ix; g1.x = U.y * ix; g1.y = U.z * ix;
            g1.z = V.x * iy; g1.w = V.y * iy; g2.x = V.z * iy;
            g2.y = W.x * iz; g2.z = W.y * iz; g2.w = W.z * iz;
            hk = log2f(ratio);
            gaussian_aabb(p, s, q, dens, b.sigma_threshold, lo, hi);
            // The boxes of the hierarchy and of the tile lists must contain the ellipsoid the per-ray test uses,
            // with room for the rounding of both tests: that ellipsoid is stretched by |q|^2 when the quaternion
            // is not a unit one (the box formula normalises it, the whitening map does not), and a ray's slab test
            // is good to a few ulp of its distance from the eye.  (The scene box, which clips the rays as in the
            // reference, is made from the unpadded boxes: bounds_kernel.)
            const float qn = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
            const float grow = fmaxf(qn, 1.0f) * 1.001f - 1.0f;
            const float3 h = make_float3(0.5f * (hi.x - lo.x), 0.5f * (hi.y - lo.y), 0.5f * (hi.z - lo.z));
            const float reach = 4e-6f * (fmaxf(fabsf(p.x), fmaxf(fabsf(p.y), fabsf(p.z))) + 1.0f);
            lo = make_float3(lo.x - (grow * h.x + reach), lo.y - (grow * h.y + reach), lo.z - (grow * h.z + reach));
            hi = make_float3(hi.x + (grow * h.x + reach), hi.y + (grow * h.y + reach), hi.z + (grow * h.z + reach));
        }
    }
    b.g0[j] = g0; b.g1[j] = g1; b.g2[j] = g2;
    b.quat[j] = qq; b.sdens[j] = sd; b.hk[j] = hk;
    b.bx[j] = make_float2(lo.x, hi.x);
    b.by[j] = make_float2(lo.y, hi.y);
    b.bz[j] = make_float2(lo.z, hi.z);
}

__global__ void fill_inverted_kernel(float2* bx, float2* by, float2* bz, int begin, int end) {
    int j = begin + blockIdx.x * blockDim.x + threadIdx.x;
    if (j < end) bx[j] = by[j] = bz[j] = make_float2(FLT_MAX, -FLT_MAX);
}

// Bottom-up refit with arrival counters: one warp per level-1 node bounds its 32
// Gaussians, then climbs; at every parent the last of the arriving children does
// the work, the others leave.  No warp ever waits for another.
__global__ void __launch_bounds__(256) refit_kernel(BuildLaunch b) {
    int node = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (node >= b.count[1]) return;
    int level = 0;
    while (true) {
        // bound children [32*node, 32*node+32) of `level` into box `node` of `level + 1`
        int c = node * kFan + lane;
        float2 x = make_float2(FLT_MAX, -FLT_MAX), y = x, z = x;
        if (c < b.count[level]) {
            int idx = b.offset[level] + c;
            x = __ldcg(&b.bx[idx]); y = __ldcg(&b.by[idx]); z = __ldcg(&b.bz[idx]);
        }
        x.x = warp_min(x.x); x.y = warp_max(x.y);
        y.x = warp_min(y.x); y.y = warp_max(y.y);
        z.x = warp_min(z.x); z.y = warp_max(z.y);
        int up = level + 1;
        if (lane == 0) {
            int idx = b.offset[up] + node;
            b.bx[idx] = x; b.by[idx] = y; b.bz[idx] = z;
        }
        if (up + 1 >= b.num_levels) return;
        int parent = node / kFan;
        int siblings = min(kFan, b.count[up] - parent * kFan);
        unsigned int arrived = 0;
        if (lane == 0) {
            __threadfence();
            arrived = atomicAdd(&b.refit_counters[b.offset[up + 1] + parent], 1u);
        }
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if ((int)arrived != siblings - 1) return;
        __threadfence();
        node = parent;
        level = up;
    }
}

}  // namespace

size_t build_cub_temp_bytes(int n_pad) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const uint64_t*)nullptr, (uint64_t*)nullptr,
                                    (const uint32_t*)nullptr, (uint32_t*)nullptr, n_pad, 0, 64, (cudaStream_t)0);
    return bytes;
}

cudaError_t launch_build(const BuildLaunch& b, cudaStream_t s) {
    const int n = b.sc.n;
    const int tb = 256;
    note_launch(), init_bounds_kernel<<<1, 32, 0, s>>>(b.bounds);
    note_launch(), bounds_kernel<<<(n + tb - 1) / tb, tb, 0, s>>>(b);
    note_launch(), morton_kernel<<<(n + tb - 1) / tb, tb, 0, s>>>(b);
    size_t temp = b.cub_temp_bytes;
    cudaError_t e = cub::DeviceRadixSort::SortPairs(b.cub_temp, temp, b.keys_in, b.keys_out, b.vals_in, b.vals_out, n,
                                                    0, 3 * b.morton_bits, s);
    if (e != cudaSuccess) return e;
    note_launch(), gather_kernel<<<(b.n_pad + tb - 1) / tb, tb, 0, s>>>(b);
    int total = b.offset[b.num_levels - 1] + ((b.count[b.num_levels - 1] + kFan - 1) / kFan) * kFan;
    int upper = total - b.offset[1];
    note_launch(), fill_inverted_kernel<<<(upper + tb - 1) / tb, tb, 0, s>>>(b.bx, b.by, b.bz, b.offset[1], total);
    e = cudaMemsetAsync(b.refit_counters, 0, sizeof(unsigned int) * (size_t)total, s);
    if (e != cudaSuccess) return e;
    int warps = b.count[1];
    note_launch(), refit_kernel<<<(warps + 7) / 8, 256, 0, s>>>(b);
    return cudaGetLastError();
}

}  // namespace rgx
