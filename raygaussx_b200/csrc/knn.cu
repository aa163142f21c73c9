// rgx_knn_mean_dist2: for every point the mean of the squared distances to its three
// nearest other points -- what the reference's point-cloud initialisation asks of
// simple-knn (classes/point_cloud.py:252,592 -> submodules/simple-knn/simple_knn.cu,
// SimpleKNN::knn) to size the first Gaussians.
//
// Exact, like the reference: points are sorted along a Morton curve, every 32
// consecutive points get a box and every 32 boxes a box of their own.  A warp owns 32
// consecutive sorted points, one query per lane; it walks the upper boxes, opens the
// ones that are nearer to some lane's query than that lane's third-best distance so
// far, and inside them the boxes of 32 points by the same rule.  The 32 points of an
// opened box are loaded with one coalesced read and handed round with shuffles.
// Queries of a warp are neighbours in space, so after the seed (the warp's own box and
// its two neighbours) nearly every box is rejected by all 32 lanes at once.
#include "rgx_internal.cuh"
#include <cub/device/device_radix_sort.cuh>

namespace rgx {

namespace {

constexpr unsigned kAll = 0xffffffffu;

__device__ __forceinline__ int ordered(float f) {          // float -> int with the same order
    int i = __float_as_int(f);
    return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float unordered(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__global__ void knn_init_kernel(int* bounds) {
    if (threadIdx.x < 3) bounds[threadIdx.x] = ordered(FLT_MAX);
    else if (threadIdx.x < 6) bounds[threadIdx.x] = ordered(-FLT_MAX);
}

__global__ void __launch_bounds__(256) knn_bounds_kernel(const float* __restrict__ pts, int n, int* bounds) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    float lo[3] = {FLT_MAX, FLT_MAX, FLT_MAX}, hi[3] = {-FLT_MAX, -FLT_MAX, -FLT_MAX};
    if (i < n)
        for (int a = 0; a < 3; ++a) lo[a] = hi[a] = pts[3 * (size_t)i + a];
    for (int a = 0; a < 3; ++a) {
        for (int o = 16; o > 0; o >>= 1) {
            lo[a] = fminf(lo[a], __shfl_xor_sync(kAll, lo[a], o));
            hi[a] = fmaxf(hi[a], __shfl_xor_sync(kAll, hi[a], o));
        }
        if ((threadIdx.x & 31) == 0) {
            atomicMin(&bounds[a], ordered(lo[a]));
            atomicMax(&bounds[3 + a], ordered(hi[a]));
        }
    }
}

__device__ __forceinline__ unsigned spread10(unsigned v) {   // 10 bits -> every third bit
    v &= 0x3ffu;
    v = (v | (v << 16)) & 0x030000ffu;
    v = (v | (v << 8)) & 0x0300f00fu;
    v = (v | (v << 4)) & 0x030c30c3u;
    v = (v | (v << 2)) & 0x09249249u;
    return v;
}

__global__ void __launch_bounds__(256) knn_keys_kernel(const float* __restrict__ pts, int n, const int* bounds,
                                                       unsigned* keys, unsigned* vals) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned q[3];
    for (int a = 0; a < 3; ++a) {
        float lo = unordered(bounds[a]), hi = unordered(bounds[3 + a]);
        float ext = hi - lo;
        float u = ext > 0.f ? (pts[3 * (size_t)i + a] - lo) / ext : 0.f;
        q[a] = (unsigned)fminf(fmaxf(u * 1023.0f, 0.f), 1023.f);
    }
    keys[i] = spread10(q[0]) | (spread10(q[1]) << 1) | (spread10(q[2]) << 2);
    vals[i] = (unsigned)i;
}

// Sorted copies of the points (w = 0), padded to a multiple of 1024 with points at infinity,
// boxes of 32 points and of 32 such boxes.  One warp per box of 32 points.
__global__ void __launch_bounds__(256) knn_gather_kernel(const float* __restrict__ pts, int n, int n_pad,
                                                         const unsigned* __restrict__ order, float4* sorted,
                                                         float4* box_lo, float4* box_hi) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int i = warp * 32 + lane;
    if (i >= n_pad) return;
    float4 p = make_float4(INFINITY, INFINITY, INFINITY, 0.f);
    if (i < n) {
        const size_t s = order[i];
        p = make_float4(pts[3 * s], pts[3 * s + 1], pts[3 * s + 2], 0.f);
    }
    sorted[i] = p;
    float lo[3] = {p.x, p.y, p.z}, hi[3] = {i < n ? p.x : -INFINITY, i < n ? p.y : -INFINITY, i < n ? p.z : -INFINITY};
    for (int a = 0; a < 3; ++a)
        for (int o = 16; o > 0; o >>= 1) {
            lo[a] = fminf(lo[a], __shfl_xor_sync(kAll, lo[a], o));
            hi[a] = fmaxf(hi[a], __shfl_xor_sync(kAll, hi[a], o));
        }
    if (lane == 0) {
        box_lo[warp] = make_float4(lo[0], lo[1], lo[2], 0.f);      // an empty box is (+inf, -inf): at infinite distance
        box_hi[warp] = make_float4(hi[0], hi[1], hi[2], 0.f);
    }
}

__global__ void __launch_bounds__(256) knn_upper_kernel(const float4* box_lo, const float4* box_hi, int n_boxes,
                                                        float4* up_lo, float4* up_hi) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int b = warp * 32 + lane;
    if (warp * 32 >= n_boxes) return;
    float4 l = b < n_boxes ? box_lo[b] : make_float4(INFINITY, INFINITY, INFINITY, 0.f);
    float4 h = b < n_boxes ? box_hi[b] : make_float4(-INFINITY, -INFINITY, -INFINITY, 0.f);
    float lo[3] = {l.x, l.y, l.z}, hi[3] = {h.x, h.y, h.z};
    for (int a = 0; a < 3; ++a)
        for (int o = 16; o > 0; o >>= 1) {
            lo[a] = fminf(lo[a], __shfl_xor_sync(kAll, lo[a], o));
            hi[a] = fmaxf(hi[a], __shfl_xor_sync(kAll, hi[a], o));
        }
    if (lane == 0) {
        up_lo[warp] = make_float4(lo[0], lo[1], lo[2], 0.f);
        up_hi[warp] = make_float4(hi[0], hi[1], hi[2], 0.f);
    }
}

// squared distance from a point to a box (0 inside; +inf for an empty box)
__device__ __forceinline__ float box_dist2(float4 lo, float4 hi, float4 p) {
    float dx = fmaxf(fmaxf(lo.x - p.x, p.x - hi.x), 0.f), dy = fmaxf(fmaxf(lo.y - p.y, p.y - hi.y), 0.f),
          dz = fmaxf(fmaxf(lo.z - p.z, p.z - hi.z), 0.f);
    return dx * dx + dy * dy + dz * dz;
}

__device__ __forceinline__ void keep3(float d, float (&best)[3]) {     // the three smallest, ascending
    if (d < best[2]) {
        if (d < best[1]) {
            best[2] = best[1];
            if (d < best[0]) { best[1] = best[0]; best[0] = d; }
            else best[1] = d;
        } else best[2] = d;
    }
}

// All lanes: measure the 32 points of box `b` against this lane's query (skipping the query itself).
__device__ __forceinline__ void open_box(const float4* __restrict__ sorted, int b, int self, float4 q, bool want,
                                         float (&best)[3], int lane) {
    const float4 mine = sorted[b * 32 + lane];
    for (int k = 0; k < 32; ++k) {
        const float x = __shfl_sync(kAll, mine.x, k), y = __shfl_sync(kAll, mine.y, k), z = __shfl_sync(kAll, mine.z, k);
        const float dx = x - q.x, dy = y - q.y, dz = z - q.z;
        const float d = dx * dx + dy * dy + dz * dz;                 // +inf for the padding points
        if (want && b * 32 + k != self) keep3(d, best);
    }
}

__global__ void __launch_bounds__(256) knn_query_kernel(const float4* __restrict__ sorted, const unsigned* __restrict__ order,
                                                        int n, int n_boxes, int n_upper, const float4* __restrict__ box_lo,
                                                        const float4* __restrict__ box_hi, const float4* __restrict__ up_lo,
                                                        const float4* __restrict__ up_hi, float* __restrict__ out) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_boxes) return;
    const int self = warp * 32 + lane;
    const bool live = self < n;
    const float4 q = sorted[self];
    float best[3] = {FLT_MAX, FLT_MAX, FLT_MAX};
    // seed: the warp's own box and its neighbours along the curve
    for (int b = max(warp - 1, 0); b <= min(warp + 1, n_boxes - 1); ++b) open_box(sorted, b, self, q, live, best, lane);
    for (int u = 0; u < n_upper; ++u) {
        const bool near_u = live && box_dist2(up_lo[u], up_hi[u], q) <= best[2];
        if (!__any_sync(kAll, near_u)) continue;
        const int b_end = min(u * 32 + 32, n_boxes);
        // this lane looks at box u*32 + lane for every query of the warp ... by turns: each lane tests its own
        // query against each of the 32 boxes, the warp opens a box if any lane wants it
        for (int b = u * 32; b < b_end; ++b) {
            if (b >= warp - 1 && b <= warp + 1) continue;            // seeded above
            const bool near_b = near_u && box_dist2(box_lo[b], box_hi[b], q) <= best[2];
            if (!__any_sync(kAll, near_b)) continue;
            open_box(sorted, b, self, q, near_b, best, lane);
        }
    }
    if (live) out[order[self]] = (best[0] + best[1] + best[2]) / 3.0f;   // simple_knn.cu: mean of the three
}

template <class T>
cudaError_t grab(T*& p, size_t count, cudaError_t prev) {
    p = nullptr;
    if (prev != cudaSuccess) return prev;
    return cudaMalloc((void**)&p, (count > 0 ? count : 1) * sizeof(T));
}

}  // namespace

}  // namespace rgx

using namespace rgx;

extern "C" RGX_API int rgx_knn_mean_dist2(int device, const float* points, int n, float* mean_dist2, rgx_stream stream) {
    if (n < 0 || (n > 0 && (!points || !mean_dist2))) return RGX_E_INVALID;
    if (n > (1 << 30)) return RGX_E_TOO_LARGE;
    if (n == 0) return RGX_OK;
    DeviceGuard guard(device);
    if (!guard.ok) { (void)cudaGetLastError(); return RGX_E_CUDA; }
    cudaStream_t s = (cudaStream_t)stream;
    const int n_pad = ((n + 1023) / 1024) * 1024;
    const int n_boxes = n_pad / 32, n_upper = n_boxes / 32;
    int* bounds; unsigned *keys_in, *keys_out, *vals_in, *vals_out; float4 *sorted, *box_lo, *box_hi, *up_lo, *up_hi;
    unsigned char* temp;
    size_t temp_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, temp_bytes, (const unsigned*)nullptr, (unsigned*)nullptr, (const unsigned*)nullptr,
                                    (unsigned*)nullptr, n, 0, 30, s);
    cudaError_t e = cudaSuccess;
    e = grab(bounds, 6, e); e = grab(keys_in, n, e); e = grab(keys_out, n, e); e = grab(vals_in, n, e); e = grab(vals_out, n, e);
    e = grab(sorted, n_pad, e); e = grab(box_lo, n_boxes, e); e = grab(box_hi, n_boxes, e); e = grab(up_lo, n_upper, e);
    e = grab(up_hi, n_upper, e); e = grab(temp, temp_bytes, e);
    if (e == cudaSuccess) {
        const int tb = 256;
        note_launch(), knn_init_kernel<<<1, 32, 0, s>>>(bounds);
        note_launch(), knn_bounds_kernel<<<(n + tb - 1) / tb, tb, 0, s>>>(points, n, bounds);
        note_launch(), knn_keys_kernel<<<(n + tb - 1) / tb, tb, 0, s>>>(points, n, bounds, keys_in, vals_in);
        e = cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys_in, keys_out, vals_in, vals_out, n, 0, 30, s);
        if (e == cudaSuccess) {
            note_launch(), knn_gather_kernel<<<(n_pad + tb - 1) / tb, tb, 0, s>>>(points, n, n_pad, vals_out, sorted, box_lo, box_hi);
            note_launch(), knn_upper_kernel<<<(n_upper * 32 + tb - 1) / tb, tb, 0, s>>>(box_lo, box_hi, n_boxes, up_lo, up_hi);
            note_launch(), knn_query_kernel<<<(n_boxes * 32 + tb - 1) / tb, tb, 0, s>>>(sorted, vals_out, n, n_boxes, n_upper, box_lo, box_hi,
                                                                      up_lo, up_hi, mean_dist2);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);       // the scratch arrays are freed below
    }
    void* all[] = {bounds, keys_in, keys_out, vals_in, vals_out, sorted, box_lo, box_hi, up_lo, up_hi, temp};
    for (void* p : all)
        if (p) cudaFree(p);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return RGX_E_CUDA; }
    return RGX_OK;
}
