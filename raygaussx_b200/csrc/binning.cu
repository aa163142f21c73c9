// Per-view tile lists.
//
// All rays of a view leave from one point, so which Gaussians a ray can meet is
// decided by where the Gaussian projects on the image.  Once per view every
// Gaussian is projected to a rectangle of 16x16-pixel tiles and paired with each
// tile it touches; the pairs are sorted by (tile, nearest distance from the eye)
// with one radix sort, and every tile ends up with a front-to-back list of
// candidate Gaussians with, per entry, the range of distances its box spans.  A ray
// then never searches the hierarchy: it slides along its tile's list.
//
// Takes the place of what OptiX traversal does for the reference at every
// optixTrace (cuda_train/forward/gaussians_aabb.cu:234-313); the list is a superset
// of every hit set, the test that decides a hit stays the per-ray one.
#include "rgx_internal.cuh"
#include "device_math.cuh"
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

namespace rgx {

namespace {

constexpr unsigned kFullMask = 0xffffffffu;

struct Projector {     // pixel coordinates of a world point: px = (a / (2 tan) + pp) * size - 0.5
    float eye[3], du[3], dv[3], dw[3];   // dual basis of (u, v, w)
    float sx, sy, ox, oy;                // px = a * sx + ox, py = b * sy + oy
};

__device__ __forceinline__ Projector make_projector(const BinLaunch& b) {
    Projector p;
    for (int k = 0; k < 3; ++k) { p.eye[k] = b.cam.eye[k]; p.du[k] = b.dual[0][k]; p.dv[k] = b.dual[1][k]; p.dw[k] = b.dual[2][k]; }
    p.sx = (float)b.cam.width / (2.0f * b.cam.tan_half_fov[0]);
    p.sy = (float)b.cam.height / (2.0f * b.cam.tan_half_fov[1]);
    p.ox = b.cam.pp[0] * (float)b.cam.width - 0.5f;
    p.oy = b.cam.pp[1] * (float)b.cam.height - 0.5f;
    return p;
}

// Camera coordinates (x right, y down, z forward, in units of the ray parametrisation a = x/z, b = y/z).
__device__ __forceinline__ void to_camera(const Projector& p, float x, float y, float z, float& xc, float& yc, float& zc) {
    float qx = x - p.eye[0], qy = y - p.eye[1], qz = z - p.eye[2];
    xc = qx * p.du[0] + qy * p.du[1] + qz * p.du[2];
    yc = qx * p.dv[0] + qy * p.dv[1] + qz * p.dv[2];
    zc = qx * p.dw[0] + qy * p.dw[1] + qz * p.dw[2];
}

// Pixel bounds of eight camera-space corners.  Returns 0 if every corner is behind
// the eye (no ray, which only goes forward, can reach the box), 1 if every corner is
// safely in front (bounds are the bounds of the projected corners), 2 otherwise.
__device__ __forceinline__ int project_corners(const Projector& p, const float* xc, const float* yc, const float* zc,
                                               float& lox, float& hix, float& loy, float& hiy) {
    bool all_front = true, all_behind = true;
    lox = loy = INFINITY; hix = hiy = -INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        float len = fabsf(xc[c]) + fabsf(yc[c]) + fabsf(zc[c]);
        bool front = zc[c] > 1e-4f * len && zc[c] > 1e-12f;
        all_front = all_front && front;
        all_behind = all_behind && !(zc[c] > 0.f);
        if (front) {
            float px = xc[c] / zc[c] * p.sx + p.ox, py = yc[c] / zc[c] * p.sy + p.oy;
            lox = fminf(lox, px); hix = fmaxf(hix, px);
            loy = fminf(loy, py); hiy = fmaxf(hiy, py);
        }
    }
    return all_behind ? 0 : (all_front ? 1 : 2);
}

// A convex body that straddles the eye plane has no bounded projection.  Its tile
// columns are found one by one instead: column [a_lo, a_hi] (in x/z) can only be
// touched if some corner lies on the inner side of each of its two bounding planes
// x - a z = 0 through the eye.  Conservative, exact per plane.  Same for rows.
__device__ __forceinline__ void straddle_tiles(const float* xc, const float* zc, float scale, float offset, int n_tiles,
                                               int tile, int n_pix, float& lo_pix, float& hi_pix) {
    lo_pix = INFINITY; hi_pix = -INFINITY;
    for (int c = 0; c < n_tiles; ++c) {
        const float p0 = (float)(c * tile), p1 = (float)min(c * tile + tile - 1, n_pix - 1);
        const float a_lo = (p0 - 0.02f - offset) / scale, a_hi = (p1 + 0.02f - offset) / scale;
        float g = -INFINITY, h = INFINITY, mag = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            g = fmaxf(g, xc[i] - a_lo * zc[i]);
            h = fminf(h, xc[i] - a_hi * zc[i]);
            mag = fmaxf(mag, fabsf(xc[i]) + (fabsf(a_lo) + fabsf(a_hi)) * fabsf(zc[i]));
        }
        if (g >= -1e-5f * mag && h <= 1e-5f * mag) { lo_pix = fminf(lo_pix, p0); hi_pix = fmaxf(hi_pix, p1); }
    }
}

__device__ __forceinline__ float3 pixel_dir(const rgx_camera& c, float px, float py) {
    float a = 2.0f * ((px + 0.5f) / (float)c.width - c.pp[0]) * c.tan_half_fov[0];
    float bq = 2.0f * ((py + 0.5f) / (float)c.height - c.pp[1]) * c.tan_half_fov[1];
    float3 d = make_float3(a * c.u[0] + bq * c.v[0] + c.w[0], a * c.u[1] + bq * c.v[1] + c.w[1],
                           a * c.u[2] + bq * c.v[2] + c.w[2]);
    float inv = 1.0f / sqrtf(dot3(d, d));
    return d * inv;
}

// Per tile: direction of the ray through the tile centre and the largest chord |d - d_c| to a
// ray of the tile (the rays of a tile lie inside the pyramid of its four corner rays).
__global__ void bin_tile_dirs_kernel(BinLaunch b, int ntiles) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= ntiles) return;
    int tx = t % b.tiles_x, ty = t / b.tiles_x + b.ty_first;
    float x0 = (float)(tx * b.tile), x1 = (float)min(tx * b.tile + b.tile - 1, b.cam.width - 1);
    float y0 = (float)(ty * b.tile), y1 = (float)min(ty * b.tile + b.tile - 1, b.cam.height - 1);
    float3 dc = pixel_dir(b.cam, 0.5f * (x0 + x1), 0.5f * (y0 + y1));
    float chord = 0.f;
    for (int c = 0; c < 4; ++c) {
        float3 d = pixel_dir(b.cam, (c & 1) ? x1 : x0, (c & 2) ? y1 : y0) - dc;
        chord = fmaxf(chord, sqrtf(dot3(d, d)));
    }
    b.tile_dir[t] = make_float4(dc.x, dc.y, dc.z, chord * 1.001f + 1e-7f);
}

// Per-Gaussian data needed to bound its meeting with a tile.
struct PairGeom {
    float2 bx, by, bz;
    float4 g0, g1, g2;
    float far_box;      // largest distance from the eye to the box
    float rho_scale;    // operator norm of the whitening map: 1 / (k s_min), with slack for non-unit quaternions
};

// Range of ray parameters at which some ray of the tile can be inside the Gaussian's box and
// inside its truncation ellipsoid; false if no ray of the tile can.  Every ray of the tile is, at
// parameter t, within t * chord of the central ray's point, so the central ray is tested against
// the box and the ellipsoid grown by that much.
__device__ __forceinline__ bool pair_range(const float* eye, float4 td, const PairGeom& g, float& tn, float& tf) {
    const float infl = g.far_box * td.w * 1.0001f + 1e-6f;
    tn = 0.f; tf = INFINITY;
    const float o[3] = {eye[0], eye[1], eye[2]}, d[3] = {td.x, td.y, td.z};
    const float lo[3] = {g.bx.x - infl, g.by.x - infl, g.bz.x - infl}, hi[3] = {g.bx.y + infl, g.by.y + infl, g.bz.y + infl};
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        if (fabsf(d[a]) < 1e-12f) {
            if (o[a] < lo[a] || o[a] > hi[a]) return false;
        } else {
            float t0 = (lo[a] - o[a]) / d[a], t1 = (hi[a] - o[a]) / d[a];
            tn = fmaxf(tn, fminf(t0, t1));
            tf = fminf(tf, fmaxf(t0, t1));
        }
    }
    if (tn > tf * (1.0f + 1e-5f) + 1e-6f) return false;
    // ellipsoid |M (x - p)| <= 1 grown to radius rho in the whitened frame
    const float rho = 1.0f + infl * g.rho_scale;
    float3 O = make_float3(o[0] - g.g0.x, o[1] - g.g0.y, o[2] - g.g0.z);
    float3 Oe = make_float3(g.g0.w * O.x + g.g1.x * O.y + g.g1.y * O.z, g.g1.z * O.x + g.g1.w * O.y + g.g2.x * O.z,
                            g.g2.y * O.x + g.g2.z * O.y + g.g2.w * O.z);
    float3 de = make_float3(g.g0.w * d[0] + g.g1.x * d[1] + g.g1.y * d[2], g.g1.z * d[0] + g.g1.w * d[1] + g.g2.x * d[2],
                            g.g2.y * d[0] + g.g2.z * d[1] + g.g2.w * d[2]);
    const float qa = dot3(de, de), qb = -dot3(Oe, de), qc = dot3(Oe, Oe) - rho * rho;
    const float disc = qb * qb - qa * qc;
    const float mag = qb * qb + fabsf(qa * qc);
    if (disc < -1e-5f * mag) return false;
    if (qa > 1e-30f) {
        const float sq = sqrtf(fmaxf(disc, 0.f) + 1e-5f * mag);
        const float r1 = (qb - sq) / qa, r2 = (qb + sq) / qa;
        tn = fmaxf(tn, r1);
        tf = fminf(tf, r2);
    }
    tn = fmaxf(tn * (1.0f - 1e-5f) - 1e-6f, 0.f);
    tf = tf * (1.0f + 1e-5f) + 1e-6f;
    return tn <= tf;
}

__device__ __forceinline__ PairGeom load_pair_geom(const BinLaunch& b, int j) {
    PairGeom g;
    g.bx = b.bx[j]; g.by = b.by[j]; g.bz = b.bz[j];
    g.g0 = b.g0[j]; g.g1 = b.g1[j]; g.g2 = b.g2[j];
    g.far_box = b.depth[j].y;
    float4 sd = b.sdens[j], q = b.quat[j];
    float k = sqrtf(2.0f * 0.6931471805599453f * b.hk[j]);
    float smin = fminf(sd.x, fminf(sd.y, sd.z));
    float qn = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
    g.rho_scale = 1.02f * fmaxf(1.0f, qn) / (k * smin);
    return g;
}

// One thread per sorted slot: tile rectangle (box rectangle cut by the rectangle of
// the oriented box of the truncation ellipsoid), distance range, number of tiles.
__global__ void __launch_bounds__(256) bin_count_kernel(BinLaunch b) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= b.n_pad) return;
    int count = 0;
    uint2 rect = make_uint2(0u, 0u);
    float2 depth = make_float2(INFINITY, -INFINITY);
    float2 bx = b.bx[j], by = b.by[j], bz = b.bz[j];
    if (j < b.n && bx.x <= bx.y) {
        const Projector p = make_projector(b);
        const int W = b.cam.width, H = b.cam.height;
        const int tiles_x_all = (W + b.tile - 1) / b.tile, tiles_y_all = (H + b.tile - 1) / b.tile;
        float xc[8], yc[8], zc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
            to_camera(p, (c & 1) ? bx.y : bx.x, (c & 2) ? by.y : by.x, (c & 4) ? bz.y : bz.x, xc[c], yc[c], zc[c]);
        float lox, hix, loy, hiy;
        int kind = project_corners(p, xc, yc, zc, lox, hix, loy, hiy);
        if (kind == 2) {
            straddle_tiles(xc, zc, p.sx, p.ox, tiles_x_all, b.tile, W, lox, hix);
            straddle_tiles(yc, zc, p.sy, p.oy, tiles_y_all, b.tile, H, loy, hiy);
        }
        if (kind != 0) {
            // oriented box of the ellipsoid {x : |S^-1 R^T (x - p)| <= k}: centre +- k s_a col_a
            float4 sd = b.sdens[j], q = b.quat[j], g0 = b.g0[j];
            float k = sqrtf(2.0f * 0.6931471805599453f * b.hk[j]) * 1.0001f;
            float3 U, V, Wc;
            quat_to_columns(q, U, V, Wc);
            float3 e0 = U * (k * sd.x), e1 = V * (k * sd.y), e2 = Wc * (k * sd.z);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float sa = (c & 1) ? 1.f : -1.f, sb = (c & 2) ? 1.f : -1.f, sc = (c & 4) ? 1.f : -1.f;
                to_camera(p, g0.x + sa * e0.x + sb * e1.x + sc * e2.x, g0.y + sa * e0.y + sb * e1.y + sc * e2.y,
                          g0.z + sa * e0.z + sb * e1.z + sc * e2.z, xc[c], yc[c], zc[c]);
            }
            float olx, ohx, oly, ohy;
            int okind = project_corners(p, xc, yc, zc, olx, ohx, oly, ohy);
            if (okind == 0) kind = 0;
            else {
                if (okind == 2) {
                    straddle_tiles(xc, zc, p.sx, p.ox, tiles_x_all, b.tile, W, olx, ohx);
                    straddle_tiles(yc, zc, p.sy, p.oy, tiles_y_all, b.tile, H, oly, ohy);
                }
                lox = fmaxf(lox, olx); hix = fminf(hix, ohx); loy = fmaxf(loy, oly); hiy = fminf(hiy, ohy);
            }
        }
        if (kind != 0) {
            // rays sit at integer pixel coordinates; keep a small safety margin for rounding
            const float m = 0.02f;
            float fx0 = ceilf(lox - m - 1e-5f * fabsf(lox)), fx1 = floorf(hix + m + 1e-5f * fabsf(hix));
            float fy0 = ceilf(loy - m - 1e-5f * fabsf(loy)), fy1 = floorf(hiy + m + 1e-5f * fabsf(hiy));
            fx0 = fmaxf(fx0, 0.f); fx1 = fminf(fx1, (float)W - 1.f);
            fy0 = fmaxf(fy0, (float)b.row_begin); fy1 = fminf(fy1, (float)b.row_end - 1.f);
            if (fx0 <= fx1 && fy0 <= fy1) {
                unsigned tx0 = (unsigned)fx0 / b.tile, tx1 = (unsigned)fx1 / b.tile;
                unsigned ty0 = (unsigned)fy0 / b.tile - b.ty_first, ty1 = (unsigned)fy1 / b.tile - b.ty_first;
                rect = make_uint2(tx0 | (tx1 << 16), ty0 | (ty1 << 16));
                count = (int)((tx1 - tx0 + 1) * (ty1 - ty0 + 1));
                float nx = fmaxf(fmaxf(bx.x - p.eye[0], p.eye[0] - bx.y), 0.f), ny = fmaxf(fmaxf(by.x - p.eye[1], p.eye[1] - by.y), 0.f),
                      nz = fmaxf(fmaxf(bz.x - p.eye[2], p.eye[2] - bz.y), 0.f);
                float fx = fmaxf(fabsf(bx.x - p.eye[0]), fabsf(bx.y - p.eye[0])), fy = fmaxf(fabsf(by.x - p.eye[1]), fabsf(by.y - p.eye[1])),
                      fz = fmaxf(fabsf(bz.x - p.eye[2]), fabsf(bz.y - p.eye[2]));
                depth.x = fmaxf(sqrtf(nx * nx + ny * ny + nz * nz) * (1.0f - 1e-5f) - 1e-6f, 0.f);
                depth.y = sqrtf(fx * fx + fy * fy + fz * fz) * (1.0f + 1e-5f) + 1e-6f;
            }
        }
    }
    b.rect[j] = rect;
    b.depth[j] = depth;
    if (count > 0) {      // keep only the tiles some ray of which can actually meet the Gaussian
        const PairGeom g = load_pair_geom(b, j);
        unsigned tx0 = rect.x & 0xffffu, tx1 = rect.x >> 16, ty0 = rect.y & 0xffffu, ty1 = rect.y >> 16;
        int kept = 0;
        for (unsigned ty = ty0; ty <= ty1; ++ty)
            for (unsigned tx = tx0; tx <= tx1; ++tx) {
                float tn, tf;
                kept += pair_range(b.cam.eye, b.tile_dir[ty * (unsigned)b.tiles_x + tx], g, tn, tf) ? 1 : 0;
            }
        count = kept;
    }
    b.counts[j] = count;
}

__global__ void bin_total_kernel(BinLaunch b) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        long long t = b.n_pad > 0 ? (long long)b.offsets[b.n_pad - 1] + b.counts[b.n_pad - 1] : 0;
        b.total_dev[0] = (int)t;
    }
}

__global__ void __launch_bounds__(256) bin_emit_kernel(BinLaunch b) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= b.n_pad) return;
    if (b.counts[j] == 0) return;
    uint2 rect = b.rect[j];
    unsigned tx0 = rect.x & 0xffffu, tx1 = rect.x >> 16, ty0 = rect.y & 0xffffu, ty1 = rect.y >> 16;
    const PairGeom g = load_pair_geom(b, j);
    size_t k = (size_t)b.offsets[j];
    for (unsigned ty = ty0; ty <= ty1; ++ty)
        for (unsigned tx = tx0; tx <= tx1; ++tx) {
            const unsigned t = ty * (unsigned)b.tiles_x + tx;
            float tn, tf;
            if (!pair_range(b.cam.eye, b.tile_dir[t], g, tn, tf)) continue;
            b.keys_in[k] = ((uint64_t)t << 32) | (uint64_t)__float_as_uint(tn);
            b.vals_in[k] = (uint32_t)k;          // emission index; the sort carries it to the pair's data
            b.pair_j[k] = j;
            b.pair_far[k] = tf;
            ++k;
        }
}

__global__ void __launch_bounds__(256) bin_ranges_kernel(BinLaunch b, int total) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= total) return;
    int t = (int)(b.keys_out[k] >> 32);
    if (k == 0 || (int)(b.keys_out[k - 1] >> 32) != t) b.tile_first[t] = k;
    if (k == total - 1 || (int)(b.keys_out[k + 1] >> 32) != t) b.tile_last[t] = k + 1;
}

__global__ void bin_tile_counts_kernel(BinLaunch b, int ntiles) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= ntiles) return;
    int cnt = b.tile_last[t] - b.tile_first[t];
    b.tile_cnt[t] = cnt;
    b.tile_pcnt[t] = ((cnt + 31) / 32) * 32;
}

__global__ void __launch_bounds__(256) bin_fill_kernel(BinLaunch b, size_t n_entries) {
    size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= n_entries) return;
    b.ent_id[k] = 0;
    b.ent_range[k] = make_float2(INFINITY, -INFINITY);
}

__global__ void __launch_bounds__(256) bin_scatter_kernel(BinLaunch b, int total) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= total) return;
    uint64_t key = b.keys_out[k];
    int t = (int)(key >> 32);
    const uint32_t src = b.vals_out[k];
    size_t dest = (size_t)b.tile_pbegin[t] + (size_t)(k - b.tile_first[t]);
    b.ent_id[dest] = b.pair_j[src];
    b.ent_range[dest] = make_float2(__uint_as_float((unsigned)(key & 0xffffffffu)), b.pair_far[src]);
}

// One warp per block of 32 entries: nearest near distance and farthest far distance.
__global__ void __launch_bounds__(256) bin_blocks_kernel(BinLaunch b, size_t n_blocks) {
    size_t blk = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (blk >= n_blocks) return;
    float2 r = b.ent_range[blk * 32 + lane];
    float lo = r.x, hi = r.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(kFullMask, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(kFullMask, hi, o));
    }
    if (lane == 0) b.blk[blk] = make_float2(lo, hi);
}

}  // namespace

size_t binning_cub_temp_bytes(size_t pair_cap, int n_pad, int ntiles) {
    size_t a = 0, c = 0, d = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, a, (const uint64_t*)nullptr, (uint64_t*)nullptr, (const uint32_t*)nullptr,
                                    (uint32_t*)nullptr, (int64_t)pair_cap, 0, 64, (cudaStream_t)0);
    cub::DeviceScan::ExclusiveSum(nullptr, c, (const int*)nullptr, (int*)nullptr, n_pad, (cudaStream_t)0);
    cub::DeviceScan::ExclusiveSum(nullptr, d, (const int*)nullptr, (int*)nullptr, ntiles + 1, (cudaStream_t)0);
    size_t m = a > c ? a : c;
    return m > d ? m : d;
}

// Phase 1: rectangles, counts, offsets, total (left in b.total_dev; the caller copies it to the host).
cudaError_t launch_bin_count(const BinLaunch& b, cudaStream_t s) {
    const int tb = 256;
    const int ntiles = b.tiles_x * b.tiles_y;
    bin_tile_dirs_kernel<<<(ntiles + tb - 1) / tb, tb, 0, s>>>(b, ntiles);
    bin_count_kernel<<<(b.n_pad + tb - 1) / tb, tb, 0, s>>>(b);
    size_t temp = b.cub_bytes;
    cudaError_t e = cub::DeviceScan::ExclusiveSum(b.cub_temp, temp, b.counts, b.offsets, b.n_pad, s);
    if (e != cudaSuccess) return e;
    bin_total_kernel<<<1, 32, 0, s>>>(b);
    return cudaGetLastError();
}

// Phase 2: emit, sort, per-tile ranges, padded layout, block summaries.
cudaError_t launch_bin_fill(const BinLaunch& b, int total, cudaStream_t s) {
    const int tb = 256;
    const int ntiles = b.tiles_x * b.tiles_y;
    cudaError_t e;
    if ((e = cudaMemsetAsync(b.tile_first, 0, sizeof(int) * (ntiles + 1), s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(b.tile_last, 0, sizeof(int) * (ntiles + 1), s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(b.tile_pcnt, 0, sizeof(int) * (ntiles + 1), s)) != cudaSuccess) return e;
    size_t temp = b.cub_bytes;
    if (total > 0) {
        bin_emit_kernel<<<(b.n_pad + tb - 1) / tb, tb, 0, s>>>(b);
        int tile_bits = 1;
        while ((1 << tile_bits) < ntiles) ++tile_bits;
        e = cub::DeviceRadixSort::SortPairs(b.cub_temp, temp, b.keys_in, b.keys_out, b.vals_in, b.vals_out, (int64_t)total, 0,
                                            32 + tile_bits, s);
        if (e != cudaSuccess) return e;
        bin_ranges_kernel<<<(total + tb - 1) / tb, tb, 0, s>>>(b, total);
    }
    bin_tile_counts_kernel<<<(ntiles + tb - 1) / tb, tb, 0, s>>>(b, ntiles);
    temp = b.cub_bytes;
    if ((e = cub::DeviceScan::ExclusiveSum(b.cub_temp, temp, b.tile_pcnt, b.tile_pbegin, ntiles + 1, s)) != cudaSuccess) return e;
    const size_t n_entries = (((size_t)total + 32u * (size_t)ntiles + 31) / 32) * 32;   // upper bound of the padded layout
    bin_fill_kernel<<<(unsigned)((n_entries + tb - 1) / tb), tb, 0, s>>>(b, n_entries);
    if (total > 0) bin_scatter_kernel<<<(total + tb - 1) / tb, tb, 0, s>>>(b, total);
    const size_t n_blocks = (n_entries + 31) / 32;
    bin_blocks_kernel<<<(unsigned)((n_blocks + 7) / 8), 256, 0, s>>>(b, n_blocks);
    return cudaGetLastError();
}

}  // namespace rgx
