// TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
//
// Host stand-ins for the handful of CUDA device built-ins that the reference's
// device sources use, so that those sources (read where they lie, never
// copied) can be compiled by g++ as plain C++ and executed on the CPU as a
// parity anchor.  Everything stays in fp32; the fast-math intrinsics map to the
// correctly rounded libm routine of the same function.
#pragma once
#include <vector_types.h>
#include <vector_functions.h>
#include <cmath>
#include <cstring>
#include <cstdint>

// glibc already declares a (non-exported) __expf, so this one has to be a macro
#define __expf(x) expf(x)
static inline float __fdividef(float a, float b) { return a / b; }
static inline float __frcp_rn(float x) { return 1.0f / x; }
static inline float rcbrtf(float x) { return 1.0f / cbrtf(x); }
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline float __int_as_float(int i) { float f; std::memcpy(&f, &i, 4); return f; }
static inline float __int_as_float(unsigned int i) { float f; std::memcpy(&f, &i, 4); return f; }
static inline int __float_as_int(float f) { int i; std::memcpy(&i, &f, 4); return i; }
template <typename T> static inline T __ldg(const T* p) { return *p; }

// Rays run on OpenMP threads in the drivers, so the gradient scatter has to be atomic.
static inline float atomicAdd(float* addr, float v) {
    float old;
#pragma omp atomic capture
    { old = *addr; *addr += v; }
    return old;
}

// Launch geometry for plain (non-OptiX) kernels; the driver sets these per emulated thread.
static thread_local uint3 threadIdx;
static thread_local uint3 blockIdx;
static thread_local dim3 blockDim;
static thread_local dim3 gridDim;
