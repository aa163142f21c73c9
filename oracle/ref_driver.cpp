// TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
//
// CPU launcher for the reference's own device sources.  The Makefile beside
// this file compiles it three times with g++, each time textually including one
// reference source from where it lies (macro REF_CU):
//   -DREF_STAGE_FORWARD   optix_raycasting/cuda_train/forward/gaussians_aabb.cu
//   -DREF_STAGE_BACKWARD  optix_raycasting/cuda_train/backward/gaussians_aabb.cu
//   -DREF_STAGE_SH        utils/sh_utils.cu
// OptiX calls resolve to optix_shim/optix.h (exhaustive-search traversal), CUDA
// built-ins to optix_shim/cuda_on_host.h.  One OpenMP thread plays one launch
// index at a time, as the 2-D OptiX launch of optix_utils.py:320 / :489 does.
// The host-side array packing that the reference performs in Python
// (optix_utils.py:268-304) is restated with numpy in oracle/ref_shim.py; this
// file only receives the packed buffers.
#include <vector>
#include <limits>
#include <omp.h>

#include REF_CU

#if defined(REF_STAGE_FORWARD) || defined(REF_STAGE_BACKWARD)

namespace {

// Per-ray superset of every later hit set: a primitive can only be reported for
// tmin >= 0 if it is reported for the query [0, +inf) (max(0,r1) <= max(tmin,r1)
// <= min(tmax,r2) <= r2), so scanning only these primitives gives the same hits
// in the same index order as scanning all of them.
void collect_candidates(unsigned int n_prims, std::vector<int>& out) {
    out.clear();
    ShimTraceState& s = shim_ts;
    s.tmin = 0.0f;
    s.tmax = std::numeric_limits<float>::infinity();
    for (unsigned int i = 0; i < n_prims; ++i) {
        s.prim = i;
        s.reported = false;
        __intersection__gaussian();
        if (s.reported) out.push_back((int)i);
    }
}

void fill_common(const float* prims, const float* bb_min, const float* bb_max, float dt_step, int dynamic_sampling,
                 int width, int height, const float* eye, const float* u, const float* v, const float* w,
                 const float* intr, int max_prim_slice, int* hit_prim_idx, float* ray_colors) {
    params.rnd_sample = 0;
    params.max_prim_slice = (unsigned int)max_prim_slice;
    params.bbox_min = make_float3(bb_min[0], bb_min[1], bb_min[2]);
    params.bbox_max = make_float3(bb_max[0], bb_max[1], bb_max[2]);
    params.dt_step = dt_step;
    params.dynamic_sampling = dynamic_sampling ? 1u : 0u;
    params.image_width = (unsigned int)width;
    params.image_height = (unsigned int)height;
    params.cam_eye = make_float3(eye[0], eye[1], eye[2]);
    params.cam_u = make_float3(u[0], u[1], u[2]);
    params.cam_v = make_float3(v[0], v[1], v[2]);
    params.cam_w = make_float3(w[0], w[1], w[2]);
    params.cam_intr = make_float4(intr[0], intr[1], intr[2], intr[3]);
    params.prims = reinterpret_cast<const PrimData*>(prims);
    params.hit_prim_idx = hit_prim_idx;
    params.ray_colors = reinterpret_cast<float3*>(ray_colors);
    params.handle = 0;
}

// stats[0..2] = optixTrace calls, intersection-program calls, reported hits (summed over rays)
void run_launch(int n_prims, int width, int height, int prefilter, int n_threads, unsigned long long* stats) {
    unsigned long long tr = 0, is = 0, rp = 0;
    if (n_threads <= 0) n_threads = omp_get_max_threads();
#pragma omp parallel num_threads(n_threads) reduction(+ : tr, is, rp)
    {
        std::vector<int> cand;
#pragma omp for schedule(dynamic, 16)
        for (int ray = 0; ray < width * height; ++ray) {
            ShimTraceState& s = shim_ts;
            s = ShimTraceState();
            s.launch_index = make_uint3((unsigned int)(ray % width), (unsigned int)(ray / width), 0u);
            s.num_prims = (unsigned int)n_prims;
            s.candidates = nullptr;
            if (prefilter) {
                float3 o, d;
                computeRay(s.launch_index, o, d);
                s.origin = o;
                s.direction = d;
                collect_candidates((unsigned int)n_prims, cand);
                s.candidates = cand.data();
                s.num_candidates = (unsigned int)cand.size();
                // an empty list must not fall back to "all primitives"
                static const int none = 0;
                if (cand.empty()) s.candidates = &none;
            }
            s.n_traces = s.n_is_calls = s.n_reports = 0;
            __raygen__rg();
            tr += s.n_traces; is += s.n_is_calls; rp += s.n_reports;
        }
    }
    if (stats) { stats[0] = tr; stats[1] = is; stats[2] = rp; }
}

}  // namespace

#endif

#if defined(REF_STAGE_FORWARD)
// ray_colors must be zero-filled by the caller, as optix_utils.py:308 does.
extern "C" int ref_forward(const float* prims, int n_prims, const float* bb_min, const float* bb_max, float dt_step,
                           int dynamic_sampling, int width, int height, const float* eye, const float* u,
                           const float* v, const float* w, const float* intr, int max_prim_slice,
                           int white_background, int* hit_prim_idx, float* ray_colors, int prefilter,
                           int n_threads, unsigned long long* stats) {
    fill_common(prims, bb_min, bb_max, dt_step, dynamic_sampling, width, height, eye, u, v, w, intr,
                max_prim_slice, hit_prim_idx, ray_colors);
    params.white_background = white_background ? 1u : 0u;
    run_launch(n_prims, width, height, prefilter, n_threads, stats);
    return 0;
}
#endif

#if defined(REF_STAGE_BACKWARD)
// The five gradient buffers are the 4-way replicated ones of optix_utils.py:471-481
// ([4N], [4N,3], [4N,3], [4N,3], [4N,4]), zero-filled by the caller.
extern "C" int ref_backward(const float* prims, int n_prims, const float* bb_min, const float* bb_max, float dt_step,
                            int dynamic_sampling, int width, int height, const float* eye, const float* u,
                            const float* v, const float* w, const float* intr, int max_prim_slice,
                            int* hit_prim_idx, float* ray_colors, float* dloss_dray_colors, float* densities_grad,
                            float* color_features_grad, float* positions_grad, float* scales_grad,
                            float* quaternions_grad, int prefilter, int n_threads, unsigned long long* stats) {
    fill_common(prims, bb_min, bb_max, dt_step, dynamic_sampling, width, height, eye, u, v, w, intr,
                max_prim_slice, hit_prim_idx, ray_colors);
    params.dloss_dray_colors = reinterpret_cast<float3*>(dloss_dray_colors);
    params.densities_grad = densities_grad;
    params.color_features_grad = reinterpret_cast<float3*>(color_features_grad);
    params.positions_grad = reinterpret_cast<float3*>(positions_grad);
    params.scales_grad = reinterpret_cast<float3*>(scales_grad);
    params.quaternions_grad = reinterpret_cast<float4*>(quaternions_grad);
    run_launch(n_prims, width, height, prefilter, n_threads, stats);
    return 0;
}
#endif

#if defined(REF_STAGE_SH)
namespace {
template <typename F>
void for_each_thread(int n, F&& body) {
    const int bs = 128;  // block size used by render_optix.py:24,44
    const int nb = (n + bs - 1) / bs;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < nb; ++b) {
        blockDim = dim3(bs, 1, 1);
        gridDim = dim3(nb, 1, 1);
        blockIdx = make_uint3((unsigned int)b, 0u, 0u);
        for (int t = 0; t < bs; ++t) {
            threadIdx = make_uint3((unsigned int)t, 0u, 0u);
            body();
        }
    }
}
}  // namespace

extern "C" int ref_forward_sh(float* campos, float* positions, float* sh, float* sg_features, float* sharpness,
                              float* lobe_axis, int num_sph_gauss, int sh_degree, int num_points, float* rgb) {
    for_each_thread(num_points, [&] {
        forward_sh(campos, reinterpret_cast<float3*>(positions), sh, sg_features, sharpness, lobe_axis,
                   (unsigned int)num_sph_gauss, sh_degree, num_points, rgb);
    });
    return 0;
}

// Output buffers zero-filled by the caller, as render_optix.py:39-43 does.
extern "C" int ref_backward_sh(float* campos, float* positions, float* sh, float* sg_features, float* sharpness,
                               float* lobe_axis, int num_sph_gauss, int sh_degree, int num_points, float* dL_drgb,
                               float* dL_dsh, float* dL_dpos, float* dL_dsg, float* dL_dsharp, float* dL_daxis) {
    for_each_thread(num_points, [&] {
        backward_sh(campos, reinterpret_cast<float3*>(positions), sh, sg_features, sharpness, lobe_axis,
                    (unsigned int)num_sph_gauss, sh_degree, num_points, reinterpret_cast<float3*>(dL_drgb), dL_dsh,
                    reinterpret_cast<float3*>(dL_dpos), dL_dsg, dL_dsharp, dL_daxis);
    });
    return 0;
}
#endif
