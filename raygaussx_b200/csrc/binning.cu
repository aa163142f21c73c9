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
#include <cub/block/block_scan.cuh>
#include <cstring>

namespace rgx {

namespace {

constexpr unsigned kFullMask = 0xffffffffu;

struct Projector {     // pixel coordinates of a world point: px = (a / (2 tan) + pp) * size - 0.5
    float eye[3], du[3], dv[3], dw[3];   // dual basis of (u, v, w)
    float sx, sy, ox, oy;                // px = a * sx + ox, py = b * sy + oy
    float plane[4][4];                   // the view's four side planes through the eye: inward normal, and its length
};

__device__ __forceinline__ Projector make_projector(const BinLaunch& b) {
    Projector p;
    for (int k = 0; k < 3; ++k) { p.eye[k] = b.cam.eye[k]; p.du[k] = b.dual[0][k]; p.dv[k] = b.dual[1][k]; p.dw[k] = b.dual[2][k]; }
    p.sx = (float)b.cam.width / (2.0f * b.cam.tan_half_fov[0]);
    p.sy = (float)b.cam.height / (2.0f * b.cam.tan_half_fov[1]);
    p.ox = b.cam.pp[0] * (float)b.cam.width - 0.5f;
    p.oy = b.cam.pp[1] * (float)b.cam.height - 0.5f;
    // a point eye + t (a u + b v + w), t > 0, of a ray of the rows at hand has a within [a0, a1] and b within [b0, b1]
    // (one pixel of margin), that is x_c - a0 z_c >= 0, a1 z_c - x_c >= 0 and the same for rows
    const float a0 = (-1.0f - p.ox) / p.sx, a1 = ((float)b.cam.width - p.ox) / p.sx;
    const float b0 = ((float)b.row_begin - 1.0f - p.oy) / p.sy, b1 = ((float)b.row_end - p.oy) / p.sy;
    for (int k = 0; k < 3; ++k) {
        p.plane[0][k] = p.du[k] - a0 * p.dw[k];
        p.plane[1][k] = a1 * p.dw[k] - p.du[k];
        p.plane[2][k] = p.dv[k] - b0 * p.dw[k];
        p.plane[3][k] = b1 * p.dw[k] - p.dv[k];
    }
    for (int q = 0; q < 4; ++q)
        p.plane[q][3] = sqrtf(p.plane[q][0] * p.plane[q][0] + p.plane[q][1] * p.plane[q][1] + p.plane[q][2] * p.plane[q][2]);
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
// columns are found from the planes through the eye instead: column [a_lo, a_hi] (in
// x/z) can only be touched if some corner lies on the inner side of each of its two
// bounding planes x - a z = 0, that is unless x_i - a_lo z_i < 0 for every corner or
// x_i - a_hi z_i > 0 for every corner.  Each of the two holds for a in an open interval
// whose ends are ratios x_i / z_i, so the eight corners are looked at once and a column
// costs two comparisons.  Conservative (a tolerance on every corner), exact per plane.
// Same for rows.  Returns the first and last pixel of the touched columns.
__device__ __forceinline__ void straddle_tiles(const float* xc, const float* zc, float scale, float offset, int n_tiles,
                                               int tile, int n_pix, float& lo_pix, float& hi_pix) {
    const float inv_scale = 1.0f / scale;
    const float a_first = (-0.02f - offset) * inv_scale, a_last = ((float)(n_pix - 1) + 0.02f - offset) * inv_scale;
    const float amax = 2.0f * fmaxf(fabsf(a_first), fabsf(a_last));
    float gl = -INFINITY, gh = INFINITY, hl = -INFINITY, hh = INFINITY;   // all below: a in (gl, gh); all above: a in (hl, hh)
    bool okg = true, okh = true;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float tol = 1e-5f * (fabsf(xc[i]) + amax * fabsf(zc[i]));
        const float up = xc[i] + tol, dn = xc[i] - tol;
        if (zc[i] > 1e-20f) {
            gl = fmaxf(gl, up / zc[i]);
            hh = fminf(hh, dn / zc[i]);
        } else if (zc[i] < -1e-20f) {
            gh = fminf(gh, up / zc[i]);
            hl = fmaxf(hl, dn / zc[i]);
        } else {
            okg = okg && up < 0.f;
            okh = okh && dn > 0.f;
        }
    }
    auto touched = [&](int c, float& p0, float& p1) {
        p0 = (float)(c * tile);
        p1 = (float)min(c * tile + tile - 1, n_pix - 1);
        const float a_lo = (p0 - 0.02f - offset) * inv_scale, a_hi = (p1 + 0.02f - offset) * inv_scale;
        const bool all_below = okg && a_lo > gl && a_lo < gh;
        const bool all_above = okh && a_hi > hl && a_hi < hh;
        return !(all_below || all_above);
    };
    lo_pix = INFINITY; hi_pix = -INFINITY;
    int c0 = 0;
    float p0, p1;
    for (; c0 < n_tiles; ++c0)
        if (touched(c0, p0, p1)) { lo_pix = p0; hi_pix = p1; break; }
    for (int c = n_tiles - 1; c > c0; --c)
        if (touched(c, p0, p1)) { hi_pix = p1; break; }
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
    const float w = chord * 1.001f + 1e-7f;
    b.tile_dir[t] = make_float4(dc.x, dc.y, dc.z, w);
    if (b.pick) atomicMax(&b.pick->chord_bits, __float_as_uint(w));      // positive floats order like their bits
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
            const float inv = __fdividef(1.0f, d[a]);      // the margins below cover its rounding
            float t0 = (lo[a] - o[a]) * inv, t1 = (hi[a] - o[a]) * inv;
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
        const float inv_qa = __fdividef(1.0f, qa);
        const float r1 = (qb - sq) * inv_qa, r2 = (qb + sq) * inv_qa;
        tn = fmaxf(tn, r1);
        tf = fminf(tf, r2);
    }
    tn = fmaxf(tn * (1.0f - 1e-5f) - 1e-6f, 0.f);
    tf = tf * (1.0f + 1e-5f) + 1e-6f;
    return tn <= tf;
}

// How a (tile, Gaussian) pair is packed into its 64-bit sort key, most significant first:
// tile | near distance (sign dropped, low mantissa bits dropped) | sorted slot of the Gaussian.
// Every key is distinct, so the sorted order does not depend on the order of emission.
// The near distance takes near_bits = 5 exponent bits + 7 to 14 mantissa bits: a window of 32 binades, 2^-16 .. 2^16
// (what lies below rounds down to zero, what lies above to the largest code), good to 0.8 % or better -- a few per
// cent of a slab's length.  The key is then as short as a whole number of 8-bit passes of the radix sort allows
// with at least 12 bits for the distance: 48 bits (six passes, not seven) for 3 M Gaussians on 4,108 tiles.
struct KeyLayout {
    int tile_bits, near_bits, id_bits;
};
constexpr int kNearExpBits = 5;
constexpr int kNearExpWindowBase = 111;     // biased exponent of 2^-16

__host__ __device__ inline KeyLayout key_layout(int ntiles, int n_pad) {
    KeyLayout k;
    k.tile_bits = 1;
    while ((1 << k.tile_bits) < ntiles) ++k.tile_bits;
    k.id_bits = 1;
    while ((1ll << k.id_bits) < (long long)n_pad) ++k.id_bits;
    const int fixed = k.tile_bits + k.id_bits;
    k.near_bits = ((fixed + 12 + 7) / 8) * 8 - fixed;            // 12 .. 19
    return k;
}

// The near distance as the list stores it: rounded down to what the key keeps, so that the
// order of the keys is exactly the order of the stored distances.
__host__ __device__ inline unsigned near_quantised(float tn, const KeyLayout& kl) {
#ifdef __CUDA_ARCH__
    const unsigned bits = __float_as_uint(tn);
#else
    unsigned bits;
    std::memcpy(&bits, &tn, sizeof(bits));
#endif
    const int mant = kl.near_bits - kNearExpBits;
    const int e = (int)((bits << 1) >> 24) - kNearExpWindowBase;
    if (e < 0) return 0u;
    if (e > 31) return (1u << kl.near_bits) - 1u;
    return ((unsigned)e << mant) | ((bits >> (23 - mant)) & ((1u << mant) - 1u));
}
__host__ __device__ inline float near_stored(unsigned q, const KeyLayout& kl) {
    const int mant = kl.near_bits - kNearExpBits;
    const unsigned bits = q == 0u ? 0u : ((((q >> mant) + (unsigned)kNearExpWindowBase) << 23) | ((q & ((1u << mant) - 1u)) << (23 - mant)));
#ifdef __CUDA_ARCH__
    return __uint_as_float(bits);
#else
    float f;
    std::memcpy(&f, &bits, sizeof(f));
    return f;
#endif
}

// Largest distance from the eye to a point of the box, rounded up (pair_range grows the box in proportion to it).
__device__ __forceinline__ float box_far_distance(const float* eye, float2 bx, float2 by, float2 bz) {
    const float fx = fmaxf(fabsf(bx.x - eye[0]), fabsf(bx.y - eye[0])), fy = fmaxf(fabsf(by.x - eye[1]), fabsf(by.y - eye[1])),
                fz = fmaxf(fabsf(bz.x - eye[2]), fabsf(bz.y - eye[2]));
    return sqrtf(fx * fx + fy * fy + fz * fz) * (1.0f + 1e-5f) + 1e-6f;
}

// What pair_range needs to know of a Gaussian, from its box, whitening map, scales, quaternion and hk.
__device__ __forceinline__ PairGeom make_pair_geom(const float* eye, float2 bx, float2 by, float2 bz, float4 g0, float4 g1,
                                                   float4 g2, float4 sd, float4 q, float kk) {
    PairGeom g;
    g.bx = bx; g.by = by; g.bz = bz;
    g.g0 = g0; g.g1 = g1; g.g2 = g2;
    g.far_box = box_far_distance(eye, bx, by, bz);
    float smin = fminf(sd.x, fminf(sd.y, sd.z));
    float qn = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
    g.rho_scale = 1.02f * fmaxf(1.0f, qn) / (kk * smin);
    return g;
}

__device__ __forceinline__ unsigned long long pair_key(const KeyLayout& kl, unsigned tile, float tn, unsigned slot) {
    return ((unsigned long long)tile << (kl.near_bits + kl.id_bits)) |
           ((unsigned long long)near_quantised(tn, kl) << kl.id_bits) | (unsigned long long)slot;
}

constexpr int kEmitThreads = 256;

// Rectangle of tiles that Gaussian j can touch: the rectangle of its box cut by the rectangle of the oriented box
// of its truncation ellipsoid.  Returns the number of tiles (0: none, rect untouched).
__device__ __forceinline__ int gaussian_rect(const BinLaunch& b, const Projector& p, int j, float2 bx, float2 by, float2 bz,
                                             uint2& rect) {
    const int W = b.cam.width, H = b.cam.height;
    const int tiles_x_all = (W + b.tile - 1) / b.tile, tiles_y_all = (H + b.tile - 1) / b.tile;
    {
        // most Gaussians lie outside the view: the sphere about the box against the four side planes
        const float cx = 0.5f * (bx.x + bx.y) - p.eye[0], cy = 0.5f * (by.x + by.y) - p.eye[1], cz = 0.5f * (bz.x + bz.y) - p.eye[2];
        const float hx = 0.5f * (bx.y - bx.x), hy = 0.5f * (by.y - by.x), hz = 0.5f * (bz.y - bz.x);
        const float r = sqrtf(hx * hx + hy * hy + hz * hz) * (1.0f + 1e-4f), far = sqrtf(cx * cx + cy * cy + cz * cz);
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (p.plane[q][0] * cx + p.plane[q][1] * cy + p.plane[q][2] * cz < -(r + 1e-5f * far + 1e-7f) * p.plane[q][3]) return 0;
    }
    float xc[8], yc[8], zc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
        to_camera(p, (c & 1) ? bx.y : bx.x, (c & 2) ? by.y : by.x, (c & 4) ? bz.y : bz.x, xc[c], yc[c], zc[c]);
    float lox, hix, loy, hiy;
    int kind = project_corners(p, xc, yc, zc, lox, hix, loy, hiy);
    if (kind == 0) return 0;
    if (kind == 2) {
        straddle_tiles(xc, zc, p.sx, p.ox, tiles_x_all, b.tile, W, lox, hix);
        straddle_tiles(yc, zc, p.sy, p.oy, tiles_y_all, b.tile, H, loy, hiy);
    }
    {
        // oriented box of the ellipsoid {x : |S^-1 R^T (x - p)| <= k}: centre +- k s_a col_a
        const float4 sd = b.sdens[j], q = b.quat[j], g0 = b.g0[j];
        const float k = sqrtf(2.0f * 0.6931471805599453f * b.hk[j]) * 1.0001f;
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
        if (okind == 0) return 0;
        if (okind == 2) {
            straddle_tiles(xc, zc, p.sx, p.ox, tiles_x_all, b.tile, W, olx, ohx);
            straddle_tiles(yc, zc, p.sy, p.oy, tiles_y_all, b.tile, H, oly, ohy);
        }
        lox = fmaxf(lox, olx); hix = fminf(hix, ohx); loy = fmaxf(loy, oly); hiy = fminf(hiy, ohy);
    }
    // rays sit at integer pixel coordinates; keep a small safety margin for rounding
    const float m = 0.02f;
    float fx0 = ceilf(lox - m - 1e-5f * fabsf(lox)), fx1 = floorf(hix + m + 1e-5f * fabsf(hix));
    float fy0 = ceilf(loy - m - 1e-5f * fabsf(loy)), fy1 = floorf(hiy + m + 1e-5f * fabsf(hiy));
    fx0 = fmaxf(fx0, 0.f); fx1 = fminf(fx1, (float)W - 1.f);
    fy0 = fmaxf(fy0, (float)b.row_begin); fy1 = fminf(fy1, (float)b.row_end - 1.f);
    if (!(fx0 <= fx1 && fy0 <= fy1)) return 0;
    const unsigned tx0 = (unsigned)fx0 / b.tile, tx1 = (unsigned)fx1 / b.tile;
    const unsigned ty0 = (unsigned)fy0 / b.tile - b.ty_first, ty1 = (unsigned)fy1 / b.tile - b.ty_first;
    rect = make_uint2(tx0 | (tx1 << 16), ty0 | (ty1 << 16));
    return (int)((tx1 - tx0 + 1) * (ty1 - ty0 + 1));
}

constexpr int kHistBits = 11;      // leading bits of the quantised near distance: its exponent bits and 3 to 6 of the mantissa
constexpr unsigned kNoRect = 0xffffffffu;

__device__ __forceinline__ unsigned hist_bucket(float tn, const KeyLayout& kl) {
    return near_quantised(tn, kl) >> (kl.near_bits - kHistBits);
}

// ---------------------------------------------------------------- culled emission
//
// Rays that end early -- those of a training view, of a dense scene -- look at the beginning of their tile's list
// only.  Such a view's lists need only hold the pairs that begin before a horizon (about near_target of them), and
// the pairs beyond need not even be emitted.  A recording forward counts the rays that reach the horizon after all
// and, if there are any, starts over with complete lists; a forward that records nothing puts those rays aside and
// takes them up again with the complete lists of their tiles (b.tile_flag) -- lists in two depths (march_lists.cu).  The horizon is picked before the emission, on the device, from what is cheap to know of a Gaussian:
// the rectangle of tiles it can touch (an upper bound of its pairs) and a lower bound of the distance at which any
// of its pairs begins.  bin_near_hist_kernel: those two per Gaussian, and their histogram; bin_pick_horizon_kernel:
// the bucket at which the running sum reaches the target; the emission kernels then skip Gaussians and pairs that
// lie in later buckets and note, per tile, that something was skipped (tile_more; for a skipped Gaussian all tiles
// of its rectangle, added up from rectangle corners by bin_tile_more_kernel).

__global__ void __launch_bounds__(kEmitThreads) bin_near_hist_kernel(BinLaunch b) {
    __shared__ unsigned int local[1 << kHistBits];
    for (int i = threadIdx.x; i < (1 << kHistBits); i += kEmitThreads) local[i] = 0u;
    __syncthreads();
    const int j = blockIdx.x * kEmitThreads + threadIdx.x;
    uint2 rect = make_uint2(kNoRect, 0u);
    unsigned code = 0u;
    if (j < b.n) {
        const float2 bx = b.bx[j], by = b.by[j], bz = b.bz[j];
        if (bx.x <= bx.y) {
            const Projector p = make_projector(b);
            const KeyLayout kl = key_layout(b.tiles_x * ((b.cam.height + b.tile - 1) / b.tile), b.n_pad);
            uint2 r;
            const int count = gaussian_rect(b, p, j, bx, by, bz, r);
            if (count > 0) {
                // No pair of this Gaussian begins before `gn`: a pair's near distance is where the tile's central ray
                // enters the box grown by far_box * chord (pair_range), a point no nearer to the eye than the box less
                // sqrt(3) times that; the margins are ten times those pair_range takes off.
                const float* e = b.cam.eye;
                const float dx = fmaxf(fmaxf(bx.x - e[0], e[0] - bx.y), 0.f), dy = fmaxf(fmaxf(by.x - e[1], e[1] - by.y), 0.f),
                            dz = fmaxf(fmaxf(bz.x - e[2], e[2] - bz.y), 0.f);
                const float infl = box_far_distance(e, bx, by, bz) * __uint_as_float(b.pick->chord_bits) * 1.0001f + 1e-6f;
                const float gn = fmaxf((sqrtf(dx * dx + dy * dy + dz * dz) - 1.7321f * infl) * (1.0f - 1e-4f) - 1e-4f, 0.f);
                code = hist_bucket(gn, kl);
                rect = r;
                atomicAdd(&local[code], (unsigned)count);
            }
        }
    }
    if (j < b.n_pad) { b.g_rect[j] = rect; b.g_code[j] = code; }
    __syncthreads();
    for (int i = threadIdx.x; i < (1 << kHistBits); i += kEmitThreads)
        if (local[i]) atomicAdd(&b.near_hist[i], (unsigned long long)local[i]);
}

// The cut: the last non-empty bucket up to which the estimated pairs stay within the target (the first non-empty
// one if none does).  Everything is kept (cut = kAllBuckets) when the view has fewer than near_min_total estimated
// pairs or the cut would keep all of them (half of them or more, with near_half).
__global__ void __launch_bounds__(1024) bin_pick_horizon_kernel(BinLaunch b) {
    using Scan = cub::BlockScan<unsigned long long, 1024>;
    __shared__ typename Scan::TempStorage scan_tmp;
    __shared__ int s_cut, s_first;
    const int t = threadIdx.x;
    const unsigned long long h0 = b.near_hist[2 * t], h1 = b.near_hist[2 * t + 1];
    unsigned long long incl, total;
    if (t == 0) { s_cut = -1; s_first = 1 << kHistBits; }
    __syncthreads();
    Scan(scan_tmp).InclusiveSum(h0 + h1, incl, total);
    const unsigned long long p0 = incl - h1, p1 = incl;
    if (h0) { atomicMin(&s_first, 2 * t); if (p0 <= b.near_target) atomicMax(&s_cut, 2 * t); }
    if (h1) { atomicMin(&s_first, 2 * t + 1); if (p1 <= b.near_target) atomicMax(&s_cut, 2 * t + 1); }
    __syncthreads();
    const int cut = s_cut >= 0 ? s_cut : s_first;
    if (t == 0) b.pick->est_total = total;
    if (cut >= (1 << kHistBits)) { if (t == 0) { b.pick->cut = kAllBuckets; b.pick->est_kept = total; } return; }
    if (t == (cut >> 1)) {
        const unsigned long long kept = (cut & 1) ? p1 : p0;
        const bool partial = total >= b.near_min_total && (b.near_half ? kept * 2 < total : kept < total) &&
                             cut + 1 < (1 << kHistBits);
        b.pick->cut = partial ? (unsigned)cut : kAllBuckets;
        b.pick->est_kept = partial ? kept : total;
    }
}

// Sorts the Gaussians into those before the cut (their slots gathered in kept_slot, so that the emission works on
// full blocks of them) and those beyond it (the corners of their rectangles go into tile_diff).
__global__ void __launch_bounds__(256) bin_compact_kernel(BinLaunch b) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const unsigned cut = b.pick->cut;
    bool keep = false;
    if (j < b.n) {
        const uint2 rect = b.g_rect[j];
        if (rect.x != kNoRect) {
            if (b.g_code[j] > cut) {                // every pair of this Gaussian begins beyond the horizon
                const unsigned tx0 = rect.x & 0xffffu, tx1 = rect.x >> 16, ty0 = rect.y & 0xffffu, ty1 = rect.y >> 16;
                const int Wd = b.tiles_x + 1;
                atomicAdd(&b.tile_diff[ty0 * Wd + tx0], 1);
                atomicAdd(&b.tile_diff[ty0 * Wd + tx1 + 1], -1);
                atomicAdd(&b.tile_diff[(ty1 + 1) * Wd + tx0], -1);
                atomicAdd(&b.tile_diff[(ty1 + 1) * Wd + tx1 + 1], 1);
            } else {
                keep = true;
            }
        }
    }
    const unsigned m = __ballot_sync(kFullMask, keep);
    if (m) {
        unsigned long long at = 0;
        if (lane == __ffs(m) - 1) at = atomicAdd(b.total_dev + 3, (unsigned long long)__popc(m));
        at = __shfl_sync(kFullMask, at, __ffs(m) - 1) + __popc(m & ((1u << lane) - 1u));
        if (keep) b.kept_slot[at] = j;
    }
}

// tile_diff holds +1 / -1 at the corners of the rectangles of the skipped Gaussians; its two-dimensional running
// sum is the number of skipped rectangles over each tile.
constexpr int kDiffShared = 12000;
__global__ void __launch_bounds__(1024) bin_tile_more_kernel(BinLaunch b) {
    __shared__ int s_diff[kDiffShared];
    const int W = b.tiles_x + 1, H = b.tiles_y + 1;
    int* d = b.tile_diff;
    if (W * H <= kDiffShared) {
        for (int i = threadIdx.x; i < W * H; i += blockDim.x) s_diff[i] = b.tile_diff[i];
        d = s_diff;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < H; r += blockDim.x) {
        int run = 0;
        for (int c = 0; c < W; ++c) { run += d[r * W + c]; d[r * W + c] = run; }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < b.tiles_x; c += blockDim.x) {
        int run = 0;
        for (int r = 0; r < b.tiles_y; ++r) {
            run += d[r * W + c];
            if (run > 0) b.tile_more[r * b.tiles_x + c] = 1;
        }
    }
}

// Complete emission, first step: every Gaussian's rectangle of tiles; those that have one are listed (big_slot,
// big_rect, their number in total_dev[1]) for bin_emit_pairs_kernel.  (A culled emission has the rectangles from
// bin_near_hist_kernel and the list from bin_compact_kernel.)
__global__ void __launch_bounds__(kEmitThreads) bin_list_kernel(BinLaunch b) {
    const int j = blockIdx.x * kEmitThreads + threadIdx.x, lane = threadIdx.x & 31;
    uint2 rect = make_uint2(kNoRect, 0u);
    bool keep = false;
    if (j < b.n) {
        const float2 bx = b.bx[j], by = b.by[j], bz = b.bz[j];
        if (bx.x <= bx.y) {
            const Projector p = make_projector(b);
            keep = gaussian_rect(b, p, j, bx, by, bz, rect) > 0;
        }
    }
    const unsigned m = __ballot_sync(kFullMask, keep);
    if (m) {
        unsigned long long at = 0;
        if (lane == __ffs(m) - 1) at = atomicAdd(b.total_dev + 1, (unsigned long long)__popc(m));
        at = __shfl_sync(kFullMask, at, __ffs(m) - 1) + __popc(m & ((1u << lane) - 1u));
        if (keep) { b.big_slot[at] = j; b.big_rect[at] = rect; }
    }
}

// The pairs of the listed Gaussians.  Warps take the Gaussians one at a time, 32 tiles of the rectangle per step:
// the tile's central ray against the box and the ellipsoid, both grown by the tile's angular radius (pair_range),
// keeps the pairs in which some ray of the tile can meet the Gaussian.  Every warp gathers its pairs in a buffer
// of its own in shared memory and appends them with one atomic per 256; pairs past the capacity are counted but
// not written (the host then grows the arrays and runs the emission again).
// An earlier version walked the candidates of 256 Gaussians block-wide, one candidate per thread whatever
// Gaussian it belonged to, and left only Gaussians of more than 48 tiles to this kernel; the search for the
// candidate's Gaussian and a block-wide barrier per round cost more than the idle lanes of small rectangles do here
// (3 M-Gaussian step by that threshold: 96: 375.9 ms, 48: 371.9, 24: 364.9, 12: 363.7, 4: 362.4, 0: 361.7).
// CULL: the list is bin_compact_kernel's; single pairs that begin beyond the cut are dropped and their tile marked.
constexpr int kBigWarps = 8;
constexpr int kBigBuf = 256;

template <bool CULL>
__global__ void __launch_bounds__(kBigWarps * 32) bin_emit_pairs_kernel(BinLaunch b) {
    const unsigned cut = CULL ? b.pick->cut : kAllBuckets;
    __shared__ unsigned long long s_keys[kBigWarps][kBigBuf];
    __shared__ float s_fars[kBigWarps][kBigBuf];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long* keys = s_keys[warp];
    float* fars = s_fars[warp];
    const unsigned long long nlisted = CULL ? b.total_dev[3] : b.total_dev[1];
    const KeyLayout kl = key_layout(b.tiles_x * ((b.cam.height + b.tile - 1) / b.tile), b.n_pad);
    int nbuf = 0;
    auto flush = [&]() {
        unsigned long long base = 0;
        if (lane == 0 && nbuf > 0) base = atomicAdd(b.total_dev, (unsigned long long)nbuf);
        base = __shfl_sync(kFullMask, base, 0);
        __syncwarp();
        for (int i = lane; i < nbuf; i += 32) {
            const unsigned long long k = base + (unsigned long long)i;
            if (k < b.pair_cap) { b.keys_in[k] = keys[i]; b.vals_in[k] = __float_as_uint(fars[i]); }
        }
        nbuf = 0;
        __syncwarp();
    };
    while (true) {
        unsigned long long idx = 0;
        if (lane == 0) idx = atomicAdd(b.total_dev + 2, 1ull);
        idx = __shfl_sync(kFullMask, idx, 0);
        if (idx >= nlisted) break;
        const int j = CULL ? b.kept_slot[idx] : b.big_slot[idx];
        const uint2 rect = CULL ? b.g_rect[j] : b.big_rect[idx];
        const float4 sd = b.sdens[j];
        const float kk = sqrtf(2.0f * 0.6931471805599453f * b.hk[j]);
        const PairGeom g = make_pair_geom(b.cam.eye, b.bx[j], b.by[j], b.bz[j], b.g0[j], b.g1[j], b.g2[j], sd, b.quat[j], kk);
        const unsigned tx0 = rect.x & 0xffffu, tx1 = rect.x >> 16, ty0 = rect.y & 0xffffu, ty1 = rect.y >> 16;
        const unsigned w = tx1 - tx0 + 1, count = w * (ty1 - ty0 + 1);
        for (unsigned it0 = 0; it0 < count; it0 += 32) {
            const unsigned item = it0 + lane;
            bool keep = false;
            unsigned long long key = 0;
            float tf = 0.f;
            if (item < count) {
                const unsigned t = (ty0 + item / w) * (unsigned)b.tiles_x + tx0 + item % w;
                float tn = 0.f;
                keep = (!b.tile_flag || b.tile_flag[t] != 0) && pair_range(b.cam.eye, b.tile_dir[t], g, tn, tf);
                if (CULL && keep && hist_bucket(tn, kl) > cut) { keep = false; b.tile_more[t] = 1; }
                if (keep) key = pair_key(kl, t, tn, (unsigned)j);
            }
            const unsigned m = __ballot_sync(kFullMask, keep);
            if (nbuf + __popc(m) > kBigBuf) flush();
            if (keep) { const int at = nbuf + __popc(m & ((1u << lane) - 1u)); keys[at] = key; fars[at] = tf; }
            nbuf += __popc(m);
        }
    }
    flush();
}

__global__ void __launch_bounds__(256) bin_ranges_kernel(BinLaunch b, int total, int tile_shift) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= total) return;
    int t = (int)(b.keys_out[k] >> tile_shift);
    if (k == 0 || (int)(b.keys_out[k - 1] >> tile_shift) != t) b.tile_first[t] = k;
    if (k == total - 1 || (int)(b.keys_out[k + 1] >> tile_shift) != t) b.tile_last[t] = k + 1;
}

__global__ void bin_tile_counts_kernel(BinLaunch b, int ntiles) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= ntiles) return;
    int cnt = b.tile_last[t] - b.tile_first[t];
    b.tile_cnt[t] = cnt;
    b.tile_pcnt[t] = ((cnt + 31) / 32) * 32;
    b.tile_iota[t] = t;
}

__global__ void __launch_bounds__(256) bin_fill_kernel(BinLaunch b, size_t n_entries) {
    size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= n_entries) return;
    b.ent_id[k] = 0;
    b.ent_range[k] = make_float2(INFINITY, -INFINITY);
}

__global__ void __launch_bounds__(256) bin_scatter_kernel(BinLaunch b, int total, KeyLayout kl) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= total) return;
    const uint64_t key = b.keys_out[k];
    const int t = (int)(key >> (kl.near_bits + kl.id_bits));
    const size_t dest = (size_t)b.tile_pbegin[t] + (size_t)(k - b.tile_first[t]);
    b.ent_id[dest] = (int)(key & ((1ull << kl.id_bits) - 1ull));
    const unsigned q = (unsigned)((key >> kl.id_bits) & ((1ull << kl.near_bits) - 1ull));
    b.ent_range[dest] = make_float2(near_stored(q, kl), __uint_as_float(b.vals_out[k]));
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

size_t binning_cub_temp_bytes(size_t pair_cap, int ntiles) {
    size_t a = 0, d = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, a, (const uint64_t*)nullptr, (uint64_t*)nullptr, (const uint32_t*)nullptr,
                                    (uint32_t*)nullptr, (int64_t)pair_cap, 0, 64, (cudaStream_t)0);
    cub::DeviceScan::ExclusiveSum(nullptr, d, (const int*)nullptr, (int*)nullptr, ntiles + 1, (cudaStream_t)0);
    size_t o = 0;
    cub::DeviceRadixSort::SortPairsDescending(nullptr, o, (const int*)nullptr, (int*)nullptr, (const int*)nullptr,
                                              (int*)nullptr, ntiles, 0, 32, (cudaStream_t)0);
    if (o > a) a = o;
    return a > d ? a : d;
}

// Phase 1: all (tile, Gaussian) pairs -- with b.pick those that begin before the horizon picked on the way --,
// unsorted, and their number in b.total_dev (which keeps counting past b.pair_cap; the caller reads it back and
// repeats the phase with more room if needed).
cudaError_t launch_bin_emit(const BinLaunch& b, cudaStream_t s) {
    const int tb = 256;
    const int ntiles = b.tiles_x * b.tiles_y;
    cudaError_t e;
    // total_dev: [0] pairs, [1] Gaussians listed by bin_list_kernel, [2] next listed Gaussian to take, [3] Gaussians
    // listed by bin_compact_kernel
    if ((e = cudaMemsetAsync(b.total_dev, 0, 4 * sizeof(unsigned long long), s)) != cudaSuccess) return e;
    const int blocks = (b.n_pad + kEmitThreads - 1) / kEmitThreads;
    if (b.pick) {
        // only the pairs that begin before a horizon, which is picked on the way (see bin_near_hist_kernel)
        const KeyLayout kl = key_layout(b.tiles_x * ((b.cam.height + b.tile - 1) / b.tile), b.n_pad);
        if (kl.near_bits < kHistBits) return cudaErrorInvalidValue;
        if ((e = cudaMemsetAsync(b.pick, 0, sizeof(HorizonPick), s)) != cudaSuccess ||
            (e = cudaMemsetAsync(b.near_hist, 0, sizeof(unsigned long long) << kHistBits, s)) != cudaSuccess ||
            (e = cudaMemsetAsync(b.tile_diff, 0, sizeof(int) * (size_t)(b.tiles_x + 1) * (size_t)(b.tiles_y + 1), s)) != cudaSuccess ||
            (e = cudaMemsetAsync(b.tile_more, 0, sizeof(int) * (size_t)ntiles, s)) != cudaSuccess)
            return e;
        note_launch(), bin_tile_dirs_kernel<<<(ntiles + tb - 1) / tb, tb, 0, s>>>(b, ntiles);
        note_launch(), bin_near_hist_kernel<<<blocks, kEmitThreads, 0, s>>>(b);
        note_launch(), bin_pick_horizon_kernel<<<1, 1024, 0, s>>>(b);
        note_launch(), bin_compact_kernel<<<(b.n_pad + 255) / 256, 256, 0, s>>>(b);
        note_launch(), bin_emit_pairs_kernel<true><<<b.big_grid, kBigWarps * 32, 0, s>>>(b);
        note_launch(), bin_tile_more_kernel<<<1, 1024, 0, s>>>(b);
        return cudaGetLastError();
    }
    note_launch(), bin_tile_dirs_kernel<<<(ntiles + tb - 1) / tb, tb, 0, s>>>(b, ntiles);
    note_launch(), bin_list_kernel<<<blocks, kEmitThreads, 0, s>>>(b);
    note_launch(), bin_emit_pairs_kernel<false><<<b.big_grid, kBigWarps * 32, 0, s>>>(b);
    return cudaGetLastError();
}

// Phase 2: sort, per-tile ranges, padded layout, block summaries.
cudaError_t launch_bin_fill(const BinLaunch& b, int total, cudaStream_t s) {
    const int tb = 256;
    const int ntiles = b.tiles_x * b.tiles_y;
    // the layout is that of the whole image whatever the row range, so that a row range sees the same order
    const KeyLayout kl = key_layout(b.tiles_x * ((b.cam.height + b.tile - 1) / b.tile), b.n_pad);
    cudaError_t e;
    if ((e = cudaMemsetAsync(b.tile_first, 0, sizeof(int) * (ntiles + 1), s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(b.tile_last, 0, sizeof(int) * (ntiles + 1), s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(b.tile_pcnt, 0, sizeof(int) * (ntiles + 1), s)) != cudaSuccess) return e;
    size_t temp = b.cub_bytes;
    if (total > 0) {
        e = cub::DeviceRadixSort::SortPairs(b.cub_temp, temp, b.keys_in, b.keys_out, b.vals_in, b.vals_out, (int64_t)total, 0,
                                            kl.tile_bits + kl.near_bits + kl.id_bits, s);
        if (e != cudaSuccess) return e;
        note_launch(), bin_ranges_kernel<<<(total + tb - 1) / tb, tb, 0, s>>>(b, total, kl.near_bits + kl.id_bits);
    }
    note_launch(), bin_tile_counts_kernel<<<(ntiles + tb - 1) / tb, tb, 0, s>>>(b, ntiles);
    temp = b.cub_bytes;
    if ((e = cub::DeviceScan::ExclusiveSum(b.cub_temp, temp, b.tile_pcnt, b.tile_pbegin, ntiles + 1, s)) != cudaSuccess) return e;
    // CTAs take the tiles with the longest lists first: the march ends with short tiles, not with one long one
    temp = b.cub_bytes;
    if ((e = cub::DeviceRadixSort::SortPairsDescending(b.cub_temp, temp, b.tile_cnt, b.tile_cnt_sorted, b.tile_iota, b.tile_order,
                                                       ntiles, 0, 32, s)) != cudaSuccess) return e;
    const size_t n_entries = (((size_t)total + 32u * (size_t)ntiles + 31) / 32) * 32;   // upper bound of the padded layout
    note_launch(), bin_fill_kernel<<<(unsigned)((n_entries + tb - 1) / tb), tb, 0, s>>>(b, n_entries);
    if (total > 0) note_launch(), bin_scatter_kernel<<<(total + tb - 1) / tb, tb, 0, s>>>(b, total, kl);
    const size_t n_blocks = (n_entries + 31) / 32;
    note_launch(), bin_blocks_kernel<<<(unsigned)((n_blocks + 7) / 8), 256, 0, s>>>(b, n_blocks);
    return cudaGetLastError();
}

// Upper end of histogram bucket `bucket` as a distance: every pair in buckets <= bucket begins before it.
float bin_hist_bucket_end(const BinLaunch& b, int bucket) {
    const KeyLayout kl = key_layout(b.tiles_x * ((b.cam.height + b.tile - 1) / b.tile), b.n_pad);
    // bucket = the leading kHistBits bits of the quantised distance; the next bucket's smallest code bounds this one
    if (bucket + 1 >= (1 << kHistBits)) return INFINITY;
    return near_stored((unsigned)(bucket + 1) << (kl.near_bits - kHistBits), kl);
}

}  // namespace rgx
