// Per-Gaussian view-dependent colour (real spherical harmonics up to degree 3 plus
// spherical-Gaussian lobes) and the gradient-finalise pass that turns the march's
// per-Gaussian gradient rows into the caller's gradient tensors.
//
// colour:   utils/sh_utils.cu:122-216 (forward_sh) fused with the rgba packing of
//           optix_raycasting/optix_utils.py:271-274
// finalise: utils/sh_utils.cu:218-412 (backward_sh) fused with the gradient
//           assembly of optix_raycasting/render_optix.py:185-199
#include "rgx_internal.cuh"
#include "device_math.cuh"

namespace rgx {

namespace {

// utils/sh_utils.cu:6-23
constexpr float kC0 = 0.28209479177387814f;
constexpr float kC1 = 0.4886025119029199f;
constexpr float kC2_0 = 1.0925484305920792f, kC2_1 = -1.0925484305920792f, kC2_2 = 0.31539156525252005f,
                kC2_3 = -1.0925484305920792f, kC2_4 = 0.5462742152960396f;
constexpr float kC3_0 = -0.5900435899266435f, kC3_1 = 2.890611442640554f, kC3_2 = -0.4570457994644658f,
                kC3_3 = 0.3731763325901154f, kC3_4 = -0.4570457994644658f, kC3_5 = 1.445305721320277f,
                kC3_6 = -0.5900435899266435f;

__device__ __forceinline__ void sh_basis(float x, float y, float z, int K, float* Y) {
    Y[0] = kC0;
    if (K > 1) { Y[1] = -kC1 * y; Y[2] = kC1 * z; Y[3] = -kC1 * x; }
    if (K > 4) {
        float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
        Y[4] = kC2_0 * xy; Y[5] = kC2_1 * yz; Y[6] = kC2_2 * (2.f * zz - xx - yy); Y[7] = kC2_3 * xz;
        Y[8] = kC2_4 * (xx - yy);
        if (K > 9) {
            Y[9] = kC3_0 * y * (3.f * xx - yy); Y[10] = kC3_1 * xy * z; Y[11] = kC3_2 * y * (4.f * zz - xx - yy);
            Y[12] = kC3_3 * z * (2.f * zz - 3.f * xx - 3.f * yy); Y[13] = kC3_4 * x * (4.f * zz - xx - yy);
            Y[14] = kC3_5 * z * (xx - yy); Y[15] = kC3_6 * x * (xx - 3.f * yy);
        }
    }
}

// d(basis)/d(dir).  `exact` selects the mathematically exact y-derivative of
// basis 9; otherwise the term coded in the reference (utils/sh_utils.cu:367).
__device__ __forceinline__ void sh_basis_grad(float x, float y, float z, int K, bool exact, float* gx, float* gy,
                                              float* gz) {
    gx[0] = gy[0] = gz[0] = 0.f;
    if (K > 1) {
        gx[1] = 0.f; gy[1] = -kC1; gz[1] = 0.f;
        gx[2] = 0.f; gy[2] = 0.f; gz[2] = kC1;
        gx[3] = -kC1; gy[3] = 0.f; gz[3] = 0.f;
    }
    if (K > 4) {
        gx[4] = kC2_0 * y; gy[4] = kC2_0 * x; gz[4] = 0.f;
        gx[5] = 0.f; gy[5] = kC2_1 * z; gz[5] = kC2_1 * y;
        gx[6] = -2.f * kC2_2 * x; gy[6] = -2.f * kC2_2 * y; gz[6] = 4.f * kC2_2 * z;
        gx[7] = kC2_3 * z; gy[7] = 0.f; gz[7] = kC2_3 * x;
        gx[8] = 2.f * kC2_4 * x; gy[8] = -2.f * kC2_4 * y; gz[8] = 0.f;
    }
    if (K > 9) {
        float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
        gx[9] = 6.f * kC3_0 * xy; gy[9] = exact ? 3.f * kC3_0 * (xx - yy) : kC3_0 * (3.f * xx - yy); gz[9] = 0.f;
        gx[10] = kC3_1 * yz; gy[10] = kC3_1 * xz; gz[10] = kC3_1 * xy;
        gx[11] = -2.f * kC3_2 * xy; gy[11] = kC3_2 * (4.f * zz - xx - 3.f * yy); gz[11] = 8.f * kC3_2 * yz;
        gx[12] = -6.f * kC3_3 * xz; gy[12] = -6.f * kC3_3 * yz; gz[12] = 3.f * kC3_3 * (2.f * zz - xx - yy);
        gx[13] = kC3_4 * (4.f * zz - 3.f * xx - yy); gy[13] = -2.f * kC3_4 * xy; gz[13] = 8.f * kC3_4 * xz;
        gx[14] = 2.f * kC3_5 * xz; gy[14] = -2.f * kC3_5 * yz; gz[14] = kC3_5 * (xx - yy);
        gx[15] = 3.f * kC3_6 * (xx - yy); gy[15] = -6.f * kC3_6 * xy; gz[15] = 0.f;
    }
}

__device__ __forceinline__ void load_row(const float* p, int K, float* out) {
    if (K == 16) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            float4 v = __ldg(p4 + t);
            out[4 * t] = v.x; out[4 * t + 1] = v.y; out[4 * t + 2] = v.z; out[4 * t + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 16; ++k) out[k] = k < K ? __ldg(p + k) : 0.f;
    }
}

__global__ void __launch_bounds__(128) colors_kernel(ColorLaunch c) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = c.sc.n;
    const int n_slots = c.perm ? ((n + 31) / 32) * 32 : n;
    if (j >= n_slots) return;
    if (c.only_if) {                     // the colours of all Gaussians after all: some ray went beyond the lists' horizon
        if (*c.only_if == 0u) return;
        if (c.listed_out) c.listed_out[j] = j < n ? 1 : 0;
    }
    if (j >= n) {
        c.rgba[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c.listed_code) c.listed_out[j] = 0;
        return;
    }
    if (c.listed_code) {
        const bool listed = !(c.listed_rect[j].x == 0xffffffffu || c.listed_code[j] > c.listed_cut);
        c.listed_out[j] = listed ? 1 : 0;
        if (!listed) return;                   // on no list of this view
    }
    const int i = c.perm ? (int)c.perm[j] : j;
    const int K = c.sc.sh_coeffs, G = c.sc.num_lobes;
    float3 v = make_float3(c.sc.positions[3 * i] - c.eye[0], c.sc.positions[3 * i + 1] - c.eye[1],
                           c.sc.positions[3 * i + 2] - c.eye[2]);
    float len = sqrtf(dot3(v, v));
    float3 d = make_float3(v.x / len, v.y / len, v.z / len);
    float rgb[3] = {0.f, 0.f, 0.f};
    for (int l = 0; l < G; ++l) {
        const float* ax = c.sc.lobe_axis + ((size_t)i * G + l) * 3;
        float sharp = c.sc.sharpness[(size_t)i * G + l];
        float lobe = expf(sharp * (d.x * ax[0] + d.y * ax[1] + d.z * ax[2] - 1.0f));
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) rgb[ch] += c.sc.sg_features[((size_t)i * 3 + ch) * G + l] * lobe;
    }
    float Y[16];
    sh_basis(d.x, d.y, d.z, K, Y);
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) {
        float row[16];
        load_row(c.sc.color_features + ((size_t)i * 3 + ch) * K, K, row);
        float acc = rgb[ch];
#pragma unroll
        for (int k = 0; k < 16; ++k)
            if (k < K) acc = fmaf(Y[k], row[k], acc);
        rgb[ch] = acc + 0.5f;
    }
    if (c.perm) {
        float dens = c.sc.densities[i];
        bool ok = dens > c.sigma_threshold;
        c.rgba[j] = ok ? make_float4(rgb[0] * dens, rgb[1] * dens, rgb[2] * dens, dens) : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        c.rgb_out[3 * i] = rgb[0]; c.rgb_out[3 * i + 1] = rgb[1]; c.rgb_out[3 * i + 2] = rgb[2];
    }
}

__device__ __forceinline__ void put(float* p, float v, bool acc) { *p = acc ? *p + v : v; }

__global__ void __launch_bounds__(128) finalize_kernel(FinalizeLaunch f) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = f.sc.n;
    if (j >= n) return;
    if (f.listed && !f.listed[j]) return;              // on no list of the view: no ray met it, its rows are clear
    const int i = (int)f.perm[j];
    const int K = f.sc.sh_coeffs, G = f.sc.num_lobes;
    const bool acc = (f.flags & RGX_FLAG_ACCUMULATE) != 0;
    const bool exact = (f.flags & RGX_FLAG_EXACT_SH_GRAD) != 0;
    float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0, r2 = r0, r3 = r0;
    for (int c = 0; c < f.grad_copies; ++c) {          // the march spreads its additions over several sets of rows
        float4* row = f.grad_rows + 4 * ((size_t)c * (size_t)f.n_pad + (size_t)j);
        const float4 a0 = row[0], a1 = row[1], a2 = row[2], a3 = row[3];
        r0.x += a0.x; r0.y += a0.y; r0.z += a0.z; r0.w += a0.w;
        r1.x += a1.x; r1.y += a1.y; r1.z += a1.z; r1.w += a1.w;
        r2.x += a2.x; r2.y += a2.y; r2.z += a2.z; r2.w += a2.w;
        r3.x += a3.x;
        // rows that received something are cleared again: every backward finds all rows clear
        const unsigned any = __float_as_uint(a0.x) | __float_as_uint(a0.y) | __float_as_uint(a0.z) | __float_as_uint(a0.w) |
                             __float_as_uint(a1.x) | __float_as_uint(a1.y) | __float_as_uint(a1.z) | __float_as_uint(a1.w) |
                             __float_as_uint(a2.x) | __float_as_uint(a2.y) | __float_as_uint(a2.z) | __float_as_uint(a2.w) |
                             __float_as_uint(a3.x) | __float_as_uint(a3.y) | __float_as_uint(a3.z) | __float_as_uint(a3.w);
        if (any) row[0] = row[1] = row[2] = row[3] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // A Gaussian no ray met (most of a large scene, in any one view) has nothing to add: the gradient tensors were
    // cleared by the launcher unless they accumulate, and are written for the others only.
    if (r0.x == 0.f && r0.y == 0.f && r0.z == 0.f && r0.w == 0.f && r1.x == 0.f && r1.y == 0.f && r1.z == 0.f &&
        r1.w == 0.f && r2.x == 0.f && r2.y == 0.f && r2.z == 0.f && r2.w == 0.f && r3.x == 0.f)
        return;
    // The march left the moments of the loss gradient in the Gaussian's whitened frame y = M (x - p),
    // M = S^-1 R^T / k (rows as in emit_global).  With N = S^-1 R^T = k M:
    //   dL/dp     = N^T k mu                      = k sum_a col_a mu_a / s_a
    //   dL/ds_a   = k^2 Y_aa / s_a
    //   dL/dcol_a = -(k^2 / s_a) sum_b Y_ab s_b row_b(R^-1),  then through the quaternion formula
    // (x - p = R^-T S k y; R^-1 has the columns of R as rows only for a unit quaternion, which nothing enforces)
    // (cuda_train/backward/gaussians_aabb.cu:401-481 summed over the samples of all rays).
    const float mu[3] = {r0.x, r0.y, r0.z};
    const float Ym[3][3] = {{r0.w, r1.z, r1.w}, {r1.z, r1.x, r2.x}, {r1.w, r2.x, r1.y}};
    const float ddens = r2.y;
    const float drgb[3] = {r2.z, r2.w, r3.x};
    const float4 sd = f.sdens[j], qq = f.quat[j];
    const float k2 = 2.0f * 0.6931471805599453f * f.hk[j];
    const float kk = sqrtf(fmaxf(k2, 0.f));
    const float sc[3] = {sd.x, sd.y, sd.z};
    float3 cols[3];
    quat_to_columns(qq, cols[0], cols[1], cols[2]);
    float3 inv_rows[3] = {cross3(cols[1], cols[2]), cross3(cols[2], cols[0]), cross3(cols[0], cols[1])};
    const float det = dot3(cols[0], inv_rows[0]);
    const float inv_det = det != 0.f ? 1.0f / det : 1.0f;
    float dpos[3] = {0.f, 0.f, 0.f};
    float dscale[3];
    float3 dcol[3];
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const float inv = 1.0f / sc[a];
        const float cf = kk * mu[a] * inv;
        dpos[0] += cols[a].x * cf; dpos[1] += cols[a].y * cf; dpos[2] += cols[a].z * cf;
        dscale[a] = k2 * Ym[a][a] * inv;
        float3 acc3 = make_float3(0.f, 0.f, 0.f);
#pragma unroll
        for (int b = 0; b < 3; ++b) acc3 = acc3 + inv_rows[b] * (Ym[a][b] * sc[b]);
        dcol[a] = acc3 * (-k2 * inv * inv_det);
    }
    const float4 dq = quat_grad_from_columns(qq, dcol[0], dcol[1], dcol[2]);
    const float dquat[4] = {dq.x, dq.y, dq.z, dq.w};
    const bool touched = r0.x != 0.f || r0.y != 0.f || r0.z != 0.f || r0.w != 0.f || r1.x != 0.f || r1.y != 0.f ||
                         r1.z != 0.f || r1.w != 0.f || r2.x != 0.f;
    if (!touched) {          // only colour or density gradients arrived: exact zeros even where hk, s or q are degenerate
        dpos[0] = dpos[1] = dpos[2] = 0.f;
        dscale[0] = dscale[1] = dscale[2] = 0.f;
    }
    const float dquat_out[4] = {touched ? dquat[0] : 0.f, touched ? dquat[1] : 0.f, touched ? dquat[2] : 0.f,
                                touched ? dquat[3] : 0.f};

#pragma unroll
    for (int a = 0; a < 3; ++a) put(f.gr.scales + 3 * (size_t)i + a, dscale[a], acc);
#pragma unroll
    for (int a = 0; a < 4; ++a) put(f.gr.quaternions + 4 * (size_t)i + a, dquat_out[a], acc);
    put(f.gr.densities + i, ddens, acc);

    const bool zero = drgb[0] == 0.f && drgb[1] == 0.f && drgb[2] == 0.f;   // utils/sh_utils.cu:226-228
    if (!zero) {                // (else the colour gradients stay as cleared, or as accumulated so far)
        float3 v = make_float3(f.sc.positions[3 * i] - f.eye[0], f.sc.positions[3 * i + 1] - f.eye[1],
                               f.sc.positions[3 * i + 2] - f.eye[2]);
        float sum2 = dot3(v, v);
        float len = sqrtf(sum2);
        float3 d = make_float3(v.x / len, v.y / len, v.z / len);
        float Y[16], gx[16], gy[16], gz[16];
        sh_basis(d.x, d.y, d.z, K, Y);
        sh_basis_grad(d.x, d.y, d.z, K, exact, gx, gy, gz);
        float ddir[3] = {0.f, 0.f, 0.f};
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
            float row[16];
            load_row(f.sc.color_features + ((size_t)i * 3 + ch) * K, K, row);
            float sx = 0.f, sy = 0.f, sz = 0.f;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (k < K) { sx = fmaf(row[k], gx[k], sx); sy = fmaf(row[k], gy[k], sy); sz = fmaf(row[k], gz[k], sz); }
            ddir[0] = fmaf(drgb[ch], sx, ddir[0]); ddir[1] = fmaf(drgb[ch], sy, ddir[1]);
            ddir[2] = fmaf(drgb[ch], sz, ddir[2]);
            float* out = f.gr.color_features + ((size_t)i * 3 + ch) * K;
            if (K == 16 && !acc) {
                float4* o4 = reinterpret_cast<float4*>(out);
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    o4[t] = make_float4(Y[4 * t] * drgb[ch], Y[4 * t + 1] * drgb[ch], Y[4 * t + 2] * drgb[ch],
                                        Y[4 * t + 3] * drgb[ch]);
            } else {
#pragma unroll
                for (int k = 0; k < 16; ++k)
                    if (k < K) put(out + k, Y[k] * drgb[ch], acc);
            }
        }
        for (int l = 0; l < G; ++l) {                                  // utils/sh_utils.cu:385-405
            const float* ax = f.sc.lobe_axis + ((size_t)i * G + l) * 3;
            float sharp = f.sc.sharpness[(size_t)i * G + l];
            float cosm1 = d.x * ax[0] + d.y * ax[1] + d.z * ax[2] - 1.0f;
            float lobe = expf(cosm1 * sharp);
            float dl_dlobe = 0.f;
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) {
                size_t o = ((size_t)i * 3 + ch) * G + l;
                put(f.gr.sg_features + o, drgb[ch] * lobe, acc);
                dl_dlobe = fmaf(drgb[ch], f.sc.sg_features[o], dl_dlobe);
            }
            float t = dl_dlobe * sharp * lobe;
            float* oa = f.gr.lobe_axis + ((size_t)i * G + l) * 3;
            put(oa, t * d.x, acc); put(oa + 1, t * d.y, acc); put(oa + 2, t * d.z, acc);
            put(f.gr.sharpness + (size_t)i * G + l, dl_dlobe * cosm1 * lobe, acc);
            ddir[0] = fmaf(t, ax[0], ddir[0]); ddir[1] = fmaf(t, ax[1], ddir[1]); ddir[2] = fmaf(t, ax[2], ddir[2]);
        }
        // through the normalisation of the view direction (utils/sh_utils.cu:406-410)
        float inv32 = 1.0f / (sum2 * len);
        float vd = v.x * ddir[0] + v.y * ddir[1] + v.z * ddir[2];
        dpos[0] += (sum2 * ddir[0] - v.x * vd) * inv32;
        dpos[1] += (sum2 * ddir[1] - v.y * vd) * inv32;
        dpos[2] += (sum2 * ddir[2] - v.z * vd) * inv32;
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) put(f.gr.positions + 3 * (size_t)i + a, dpos[a], acc);
}

}  // namespace

cudaError_t launch_colors(const ColorLaunch& c, cudaStream_t s) {
    int slots = c.perm ? ((c.sc.n + 31) / 32) * 32 : c.sc.n;
    if (slots == 0) return cudaSuccess;
    note_launch(), colors_kernel<<<(slots + 127) / 128, 128, 0, s>>>(c);
    return cudaGetLastError();
}

cudaError_t launch_finalize(const FinalizeLaunch& f, cudaStream_t s) {
    if (f.sc.n == 0) return cudaSuccess;
    if (!(f.flags & RGX_FLAG_ACCUMULATE)) {       // the kernel writes the rows of the Gaussians some ray met, nothing else
        const size_t n = (size_t)f.sc.n, K = (size_t)f.sc.sh_coeffs, G = (size_t)f.sc.num_lobes;
        struct { float* p; size_t count; } clear[] = {
            {f.gr.positions, 3 * n}, {f.gr.scales, 3 * n}, {f.gr.quaternions, 4 * n}, {f.gr.densities, n},
            {f.gr.color_features, 3 * K * n}, {f.gr.sg_features, 3 * G * n}, {f.gr.sharpness, G * n},
            {f.gr.lobe_axis, 3 * G * n}};
        for (auto& c : clear) {
            if (!c.p || c.count == 0) continue;
            cudaError_t e = cudaMemsetAsync(c.p, 0, c.count * sizeof(float), s);
            if (e != cudaSuccess) return e;
        }
    }
    note_launch(), finalize_kernel<<<(f.sc.n + 127) / 128, 128, 0, s>>>(f);
    return cudaGetLastError();
}

}  // namespace rgx
