// TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
//
// A CPU stand-in for the few OptiX 7 device-API calls made by the reference's
// ray-marching programs.  OptiX itself (closed source, needs RT-capable driver
// components) cannot be had offline, but the *result* of a trace is fixed by
// the reference's own programs: the hit set of a query [tmin, tmax] is the set
// of primitives whose intersection program reports a hit, the closest hit is
// the smallest reported t, and the any-hit program sees every reported hit
// until it terminates the ray.  So traversal is replaced here by an exhaustive
// loop over primitives (optionally over a per-ray candidate list that the
// driver proved to be a superset), and the reference's programs are called
// exactly as the OptiX runtime would call them:
//
//   optixTrace -> for each primitive: __intersection__gaussian
//                   -> optixReportIntersection (accepted iff tmin <= t <= current tmax)
//                        -> any-hit program (hit group 1 only, unless disabled by ray flag)
//                             optixIgnoreIntersection: hit is dropped, tmax unchanged
//                             optixTerminateRay: hit is committed, traversal stops
//                        -> otherwise the hit is committed and tmax shrinks to t
//              -> closest-hit program (hit group 0, unless disabled) or miss program
//
// The order in which OptiX presents primitives is implementation defined; the
// loop below uses index order.  Results only depend on that order when a slab
// holds more hits than max_prim_slice.
#pragma once
#include "cuda_on_host.h"

typedef unsigned long long OptixTraversableHandle;
typedef unsigned int OptixVisibilityMask;

enum OptixRayFlagsShim {
    OPTIX_RAY_FLAG_NONE = 0u,
    OPTIX_RAY_FLAG_DISABLE_ANYHIT = 1u << 0,
    OPTIX_RAY_FLAG_ENFORCE_ANYHIT = 1u << 1,
    OPTIX_RAY_FLAG_TERMINATE_ON_FIRST_HIT = 1u << 2,
    OPTIX_RAY_FLAG_DISABLE_CLOSESTHIT = 1u << 3,
};

// Programs defined by the reference translation unit that includes this header.
extern "C" void __intersection__gaussian();
extern "C" void __anyhit__ah();
extern "C" void __closesthit__ch();
extern "C" void __miss__ms_ch();
extern "C" void __miss__ms_ah();

struct ShimTraceState {
    uint3 launch_index;
    float3 origin, direction;
    float tmin, tmax;
    unsigned int prim;
    unsigned int payload0;
    bool reported, ignored, terminated;
    float reported_t;
    // primitives to visit: all of [0, num_prims) or an explicit candidate list
    unsigned int num_prims;
    const int* candidates;
    unsigned int num_candidates;
    // bookkeeping for the work counters of the test-suite
    unsigned long long n_traces, n_is_calls, n_reports;
};
static thread_local ShimTraceState shim_ts;

static inline uint3 optixGetLaunchIndex() { return shim_ts.launch_index; }
static inline unsigned int optixGetPrimitiveIndex() { return shim_ts.prim; }
static inline float3 optixGetWorldRayDirection() { return shim_ts.direction; }
static inline float3 optixGetWorldRayOrigin() { return shim_ts.origin; }
static inline float optixGetRayTmin() { return shim_ts.tmin; }
static inline float optixGetRayTmax() { return shim_ts.tmax; }
static inline unsigned int optixGetPayload_0() { return shim_ts.payload0; }
static inline void optixSetPayload_0(unsigned int v) { shim_ts.payload0 = v; }
static inline void optixSetPayload_0(int v) { shim_ts.payload0 = (unsigned int)v; }
static inline void optixIgnoreIntersection() { shim_ts.ignored = true; }
static inline void optixTerminateRay() { shim_ts.terminated = true; }

static inline bool optixReportIntersection(float t, unsigned int /*kind*/) {
    if (!(t >= shim_ts.tmin && t <= shim_ts.tmax)) return false;
    shim_ts.reported = true;
    shim_ts.reported_t = t;
    return true;
}

static inline void optixTrace(OptixTraversableHandle, float3 origin, float3 direction, float tmin, float tmax,
                              float /*rayTime*/, OptixVisibilityMask, unsigned int rayFlags,
                              unsigned int sbtOffset, unsigned int /*sbtStride*/, unsigned int missIndex,
                              unsigned int& p0) {
    ShimTraceState& s = shim_ts;
    s.origin = origin; s.direction = direction; s.tmin = tmin; s.tmax = tmax;
    s.payload0 = p0; s.terminated = false;
    s.n_traces++;
    bool committed = false;
    const bool has_anyhit = (sbtOffset == 1u) && !(rayFlags & OPTIX_RAY_FLAG_DISABLE_ANYHIT);
    const unsigned int n = s.candidates ? s.num_candidates : s.num_prims;
    for (unsigned int i = 0; i < n; ++i) {
        s.prim = s.candidates ? (unsigned int)s.candidates[i] : i;
        s.reported = false;
        s.n_is_calls++;
        __intersection__gaussian();
        if (!s.reported) continue;
        s.n_reports++;
        if (has_anyhit) {
            s.ignored = false;
            __anyhit__ah();
            if (s.ignored) continue;
        }
        committed = true;
        s.tmax = s.reported_t;
        if (s.terminated) break;
    }
    if (!committed) {
        if (missIndex == 0u) __miss__ms_ch(); else __miss__ms_ah();
    } else if (sbtOffset == 0u && !(rayFlags & OPTIX_RAY_FLAG_DISABLE_CLOSESTHIT)) {
        __closesthit__ch();
    }
    p0 = s.payload0;
}
