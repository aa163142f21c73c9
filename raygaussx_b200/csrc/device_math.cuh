// Small fp32 device helpers shared by the kernels.
#pragma once
#include <cuda_runtime.h>
#include <math.h>

namespace rgx {

__device__ __forceinline__ float3 operator+(float3 a, float3 b) { return make_float3(a.x + b.x, a.y + b.y, a.z + b.z); }
__device__ __forceinline__ float3 operator-(float3 a, float3 b) { return make_float3(a.x - b.x, a.y - b.y, a.z - b.z); }
__device__ __forceinline__ float3 operator*(float3 a, float s) { return make_float3(a.x * s, a.y * s, a.z * s); }
__device__ __forceinline__ float3 operator*(float s, float3 a) { return make_float3(a.x * s, a.y * s, a.z * s); }
__device__ __forceinline__ float dot3(float3 a, float3 b) { return fmaf(a.x, b.x, fmaf(a.y, b.y, a.z * b.z)); }
__device__ __forceinline__ float3 cross3(float3 a, float3 b) {
    return make_float3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}

// Columns (U, V, W) of the rotation given by the un-normalised quaternion formula
// the reference uses for intersection and marching
// (cuda_train/forward/gaussians_aabb.cu:7-17); q = (w, x, y, z) with vector part v = (x, y, z).
// Written as R = I - (tr(S) I - S) + A with the symmetric part S = 2 v v^T and the antisymmetric part
// A = 2 w [v]_x, which for a unit quaternion is the usual rotation and for any other the same
// polynomial the reference evaluates.
__device__ __forceinline__ void quat_to_columns(float4 q, float3& U, float3& V, float3& W) {
    const float w = q.x;
    const float3 v = make_float3(q.y, q.z, q.w);
    const float3 v2 = make_float3(v.x + v.x, v.y + v.y, v.z + v.z);
    const float3 diag = make_float3(v.x * v2.x, v.y * v2.y, v.z * v2.z);       // S_xx, S_yy, S_zz
    const float3 off = make_float3(v.y * v2.z, v.x * v2.z, v.x * v2.y);        // S_yz, S_xz, S_xy
    const float3 anti = make_float3(w * v2.x, w * v2.y, w * v2.z);             // A_zy, A_xz, A_yx
    U = make_float3(1.f - (diag.y + diag.z), off.z + anti.z, off.y - anti.y);
    V = make_float3(off.z - anti.z, 1.f - (diag.x + diag.z), off.x + anti.x);
    W = make_float3(off.y + anti.y, off.x - anti.x, 1.f - (diag.x + diag.y));
}

// Gradient of the same formula w.r.t. q given the gradients of the three columns
// (cuda_train/backward/gaussians_aabb.cu:469-481).
__device__ __forceinline__ float4 quat_grad_from_columns(float4 q, float3 dU, float3 dV, float3 dW) {
    const float r = q.x, i = q.y, j = q.z, k = q.w;
    float4 g;
    g.x = 2.f * (k * dU.y - j * dU.z - k * dV.x + i * dV.z + j * dW.x - i * dW.y);
    g.y = 2.f * (j * dU.y + k * dU.z + j * dV.x - 2.f * i * dV.y + r * dV.z + k * dW.x - r * dW.y - 2.f * i * dW.z);
    g.z = 2.f * (-2.f * j * dU.x + i * dU.y - r * dU.z + i * dV.x + k * dV.z + r * dW.x + k * dW.y - 2.f * j * dW.z);
    g.w = 2.f * (-2.f * k * dU.x + r * dU.y + i * dU.z - r * dV.x - 2.f * k * dV.y + j * dV.z + i * dW.x + j * dW.y);
    return g;
}

// Box of the sigma_threshold iso-ellipsoid (optix_raycasting/optix_utils.py:48-77):
// the quaternion is renormalised here, and a Gaussian at or below the threshold
// gets a zero-size box at its centre.
__device__ __forceinline__ void gaussian_aabb(float3 c, float3 s, float4 q, float dens, float sigma_threshold,
                                              float3& lo, float3& hi) {
    float t = dens / sigma_threshold;
    float d = logf(t * t);
    if (!(d > 0.0f)) d = 0.0f;
    d = sqrtf(d);
    float W = q.x, X = q.y, Y = q.z, Z = q.w;
    float n = W * W + X * X + Y * Y + Z * Z;
    float invn = rsqrtf(n + 1e-20f);
    W *= invn; X *= invn; Y *= invn; Z *= invn;
    float L1x = 1.f - 2.f * (Y * Y + Z * Z), L1y = 2.f * (X * Y - W * Z), L1z = 2.f * (X * Z + W * Y);
    float L2x = 2.f * (X * Y + W * Z), L2y = 1.f - 2.f * (X * X + Z * Z), L2z = 2.f * (Y * Z - W * X);
    float L3x = 2.f * (X * Z - W * Y), L3y = 2.f * (Y * Z + W * X), L3z = 1.f - 2.f * (X * X + Y * Y);
    float hx = d * sqrtf((s.x * L1x) * (s.x * L1x) + (s.y * L1y) * (s.y * L1y) + (s.z * L1z) * (s.z * L1z));
    float hy = d * sqrtf((s.x * L2x) * (s.x * L2x) + (s.y * L2y) * (s.y * L2y) + (s.z * L2z) * (s.z * L2z));
    float hz = d * sqrtf((s.x * L3x) * (s.x * L3x) + (s.y * L3y) * (s.y * L3y) + (s.z * L3z) * (s.z * L3z));
    lo = make_float3(c.x - hx, c.y - hy, c.z - hz);
    hi = make_float3(c.x + hx, c.y + hy, c.z + hz);
}

__device__ __forceinline__ float sqrt_approx(float x) {
    float y;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace rgx
