/*
 * rgx -- differentiable Gaussian ray marching for NVIDIA B200 (sm_100a).
 *
 * C ABI of the shared library librgx.so.  It replaces, for one device, what the
 * reference renderer does between its autograd boundary and the GPU: bounding
 * boxes, acceleration-structure build, per-view colour evaluation, the forward
 * ray march and the backward ray march with all gradient reductions.
 *
 * Conventions
 *   - every pointer named in a struct or argument list is a DEVICE pointer to
 *     contiguous fp32 (or int32) data owned by the caller, unless stated;
 *   - rgx_scene.quaternions must start on a 16-byte boundary, and so must
 *     rgx_scene.color_features and rgx_grads.color_features when sh_coeffs is 16
 *     (the kernels move them 16 bytes at a time); anything else is refused with
 *     RGX_E_INVALID before a kernel is launched.  Whole allocations of cudaMalloc
 *     or of a framework's allocator satisfy this; a row slice of one may not;
 *   - every call enqueues its work on the given CUDA stream and returns without
 *     synchronising, and performs no device->host copy, unless its comment says
 *     otherwise (rgx_forward and rgx_backward do say otherwise: see there);
 *   - return value 0 is success, negative values are RGX_E_*; nothing throws;
 *   - every call makes its device current while it runs and puts the caller's
 *     current device back before it returns;
 *   - a context belongs to one device and one host thread at a time;
 *   - the context owns its workspace (device memory grown on demand in
 *     rgx_build / rgx_forward / rgx_backward, freed in rgx_destroy).
 */
#ifndef RGX_H
#define RGX_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define RGX_API __attribute__((visibility("default")))
#else
#define RGX_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rgx_ctx rgx_ctx;
typedef void* rgx_stream; /* a cudaStream_t */

enum {
    RGX_OK = 0,
    RGX_E_INVALID = -1, /* bad argument (null pointer, negative size, unsupported SH count ...) */
    RGX_E_CUDA = -2,    /* a CUDA runtime call failed; see rgx_last_error */
    RGX_E_NOT_BUILT = -3, /* rgx_forward / rgx_backward before rgx_build, or with a different Gaussian count */
    RGX_E_TOO_LARGE = -4  /* size beyond a fixed capacity (see the call's comment) */
};

/* The Gaussian set: the eight tensors the reference operator receives
 * (optix_raycasting/render_optix.py:94-95), produced by PointCloud.get_data
 * (classes/point_cloud.py:549-559). */
typedef struct rgx_scene {
    int32_t n;              /* number of Gaussians */
    int32_t sh_coeffs;      /* coefficients per channel, (degree+1)^2: 1, 4, 9 or 16 */
    int32_t num_lobes;      /* spherical-Gaussian lobes per Gaussian (0..8) */
    const float* positions;      /* [n,3] */
    const float* scales;         /* [n,3] already exponentiated */
    const float* quaternions;    /* [n,4] (w,x,y,z), used as given (not renormalised) */
    const float* densities;      /* [n]   raw; Gaussians with density <= sigma_threshold never contribute */
    const float* color_features; /* [n,3,sh_coeffs] channel-major */
    const float* sg_features;    /* [n,3,num_lobes] or NULL when num_lobes == 0 */
    const float* sharpness;      /* [n,num_lobes] */
    const float* lobe_axis;      /* [n,num_lobes,3] */
} rgx_scene;

/* Pinhole camera: the launch-parameter fields of optix_raycasting/optix_utils.py:258-266. */
typedef struct rgx_camera {
    float eye[3];          /* camera_center */
    float u[3], v[3], w[3];/* columns 0,1,2 of world_view_transform[:3,:3]: camera x (right), y (down), z (forward) */
    float tan_half_fov[2]; /* tan(FoVx/2), tan(FoVy/2) */
    float pp[2];           /* principal point as a fraction of the image (0.5 = centre) */
    int32_t width, height; /* in rays: image size times supersampling */
} rgx_camera;

/* Marching parameters: Params of cuda_train/forward/gaussians_aabb.h:14-44 plus the
 * constants of :2-5 that a caller may need to vary. */
typedef struct rgx_march {
    float dt_step;
    int32_t dynamic_sampling;
    int32_t max_prim_slice;    /* hit cap per 32-sample slab; further hits of that slab are dropped and counted */
    int32_t white_background;
    float transmittance_eps;   /* 1e-3 in the reference */
    int32_t row_begin, row_end;/* image rows [row_begin,row_end) to march; rays outside are left untouched */
    int32_t flags;             /* RGX_FLAG_* */
} rgx_march;

enum {
    RGX_FLAG_COUNT_WORK = 1,     /* also accumulate the work counters read by rgx_read_counters */
    RGX_FLAG_BRUTE_FORCE = 2,    /* skip the hierarchy: test every Gaussian in every query (validation only) */
    RGX_FLAG_EXACT_SH_GRAD = 4,  /* backward: exact d(basis 9)/dy instead of the reference's term (utils/sh_utils.cu:367) */
    RGX_FLAG_ACCUMULATE = 8,     /* backward: add into the gradient tensors instead of overwriting them */
    RGX_FLAG_SAVE_HITS = 32,     /* forward: keep, per ray and slab, the Gaussians that were hit and the per-sample
                                    sums (in the context's workspace, about 3 KB per ray) so that a backward for
                                    the same view replays them instead of searching and evaluating again; the
                                    backward falls back to searching where nothing was kept */
    RGX_FLAG_PER_RAY_SEARCH = 16 /* search the hierarchy once per ray and slab instead of sliding along the view's
                                    per-tile lists (same hits; the general path, kept for validation and used by
                                    rgx_forward_static) */
};

/* Gradient tensors, shaped like the inputs (what RenderOptixFunction.backward
 * returns, render_optix.py:199).  sg_* may be NULL when num_lobes == 0. */
typedef struct rgx_grads {
    float* positions;      /* [n,3] march gradient plus the view-direction term */
    float* scales;         /* [n,3] w.r.t. the exponentiated scales */
    float* quaternions;    /* [n,4] derivative of the un-normalised rotation formula */
    float* densities;      /* [n] */
    float* color_features; /* [n,3,sh_coeffs] */
    float* sg_features;    /* [n,3,num_lobes] */
    float* sharpness;      /* [n,num_lobes] */
    float* lobe_axis;      /* [n,num_lobes,3] */
} rgx_grads;

/* Work counters summed over the rays marched since the last reset (host struct). */
typedef struct rgx_counters {
    uint64_t rays;          /* rays marched */
    uint64_t slabs;         /* S: slab iterations */
    uint64_t slabs_hit;     /* S_h: slabs with at least one hit */
    uint64_t closest_queries;/* Q_c: closest-hit queries */
    uint64_t hits;          /* P: hit-list entries summed over slabs */
    uint64_t pairs_inside;  /* E_in: (sample, Gaussian) pairs inside the truncation ellipsoid */
    uint64_t overflow_slabs;/* OVF: slabs that reached max_prim_slice */
    uint64_t node_tests;    /* box tests against hierarchy nodes (32 per warp step) */
    uint64_t prim_tests;    /* box tests against Gaussians */
    uint64_t ellipsoid_tests;/* exact ray/ellipsoid tests */
    uint64_t stack_overflows;/* traversal-stack overflows (results invalid if non-zero) */
    uint64_t hits_hash;     /* order-independent hash of every (ray, slab, Gaussian) hit triple */
    uint64_t candidates;    /* tile-list march: list entries looked at (32 per opened block of a tile's list) */
    /* tile-list forward march, counting variant: warp-cycles spent per phase (clock64 differences summed over
     * warps).  cycles_search contains cycles_wait, which contains cycles_window and most of cycles_eval. */
    uint64_t cycles_window;   /* staging of hits for the evaluation */
    uint64_t cycles_seek;     /* closest-hit queries over the tile's list */
    uint64_t cycles_search;   /* slab queries: list scan, exact tests, staging, evaluation */
    uint64_t cycles_eval;     /* per-sample evaluation of staged Gaussians */
    uint64_t cycles_composite;/* compositing of a slab */
    uint64_t cycles_wait;     /* exact tests of 32 candidates and what follows from their hits */
    uint64_t cycles_total;    /* whole ray */
} rgx_counters;

/* Replaces: ox.DeviceContext / module / pipeline creation (optix_utils.py:154-210). */
RGX_API int rgx_create(int device, rgx_ctx** out);
RGX_API void rgx_destroy(rgx_ctx* ctx);
/* Host string describing the last failure on this context (never NULL). */
RGX_API const char* rgx_last_error(const rgx_ctx* ctx);

enum {
    RGX_CURVE_MORTON = 0, /* Z-order keys */
    RGX_CURVE_HILBERT = 1 /* Hilbert-curve keys: same cost to sort, tighter groups */
};

/* Replaces: ellipsoids_bbox_from_quat + create_acceleration_structure
 * (optix_utils.py:82-109,139-142; called from render_optix.py:109-117).
 * Computes per-Gaussian boxes of the sigma_threshold iso-ellipsoid, the scene box,
 * 3*key_bits-bit space-filling-curve keys of the centres (key_bits per axis: 10
 * or 20; curve: RGX_CURVE_*), sorts them (CUB radix sort) and refits a 32-ary
 * hierarchy bottom-up.  Only positions,
 * scales, quaternions and densities of `scene` are read.  Must be called again
 * whenever one of those four tensors changes. */
RGX_API int rgx_build(rgx_ctx* ctx, const rgx_scene* scene, float sigma_threshold, int key_bits, int curve,
                      rgx_stream stream);

/* Replaces: compute_cupy_rgb + launch_pipeline_forward (render_optix.py:121-131;
 * device code cuda_train/forward/gaussians_aabb.cu, utils/sh_utils.cu:122-216).
 * rgb [R,3] is required; alpha [R] (1 - final transmittance) and depth [R]
 * (expected depth, cuda_gui/gaussians_aabb.cu:189-202) may be NULL.  R = width*height.
 * Host synchronisation: the first forward (or backward) of a view -- a camera and row range for which the
 * context holds no tile lists yet -- waits once on `stream` for the number of (tile, Gaussian) pairs of the
 * view (8 bytes device->host), which sizes the sort; a forward-only view that takes the two-depth path
 * (rgx_debug_two_depth) waits up to three times.  A view whose lists were made ahead (rgx_hint_next_view) or
 * are still cached does not wait.  RGX_FLAG_PER_RAY_SEARCH and RGX_FLAG_BRUTE_FORCE never wait. */
RGX_API int rgx_forward(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march,
                float* rgb, float* alpha, float* depth, rgx_stream stream);

/* Replaces: the viewer's ray generation program with its frame and depth buffers
 * (cuda_gui/gaussians_aabb.cu:205-342; colour quantisation cuda_gui/helpers.h:45-58:
 * clamp to [0,1], times 256, truncated, at most 255, no gamma; alpha byte 255).
 * Same march as rgx_forward; frame_rgba8 is [R,4] bytes in a plain device buffer
 * (no window, swapchain or graphics interop), depth [R] may be NULL.  The viewer
 * composites over black: pass white_background = 0 for its exact output. */
RGX_API int rgx_forward_frame(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march,
                              unsigned char* frame_rgba8, float* depth, rgx_stream stream);

/* Replaces: launch_pipeline_backward + reduce_temp_grads + compute_cupy_sh_grad
 * (render_optix.py:166-185; device code cuda_train/backward/gaussians_aabb.cu,
 * utils/sh_utils.cu:218-412).  rgb is the forward's output for the same camera,
 * dL_drgb [R,3] the incoming gradient; rays outside [row_begin,row_end) are not read.
 * The geometry (positions, scales, quaternions, densities) is NOT read from `scene` here but from the
 * context's latest rgx_build: call rgx_backward before any rgx_build with other values, or build again from
 * the forward's tensors first (a recording made before that build is then ignored and the rays are searched
 * again).  `scene` supplies the count, the colour tensors and the shapes of the gradients.
 * Host synchronisation: as rgx_forward, when the view's lists have to be made; and, when the lists of an
 * announced next view are made beside it, one wait on a stream of the context's own (not on `stream`). */
RGX_API int rgx_backward(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march,
                 const float* rgb, const float* dL_drgb, const rgx_grads* grads, rgx_stream stream);

/* Announces the view of the next rgx_forward (no counterpart in the reference, where OptiX traversal needs no
 * per-view preparation).  The rgx_backward that follows makes that view's tile lists on a stream of the context's
 * own, beside its replay of the recording and the gradient assembly, which read no lists; the announced forward
 * then finds them made (it waits for them on its stream).  Purely an optimisation: results are those of the
 * calls without it, a wrong announcement costs one unused list construction.  The announcement holds for one
 * rgx_backward; NULL, NULL withdraws it.  rgx_lists_made_ahead: how many lists were made this way so far. */
RGX_API int rgx_hint_next_view(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* march);
RGX_API int rgx_lists_made_ahead(const rgx_ctx* ctx);

/* Per-Gaussian view-dependent colour only (render_optix.py:19-32): rgb_out [n,3]
 * in the caller's Gaussian order. */
RGX_API int rgx_gaussian_colors(rgx_ctx* ctx, const rgx_scene* scene, const float eye[3], float* rgb_out,
                        rgx_stream stream);

/* Scene box computed by the last rgx_build, copied to host (synchronises the stream). */
RGX_API int rgx_scene_box(rgx_ctx* ctx, float bb_min[3], float bb_max[3], rgx_stream stream);

/* Work counters (RGX_FLAG_COUNT_WORK).  rgx_read_counters synchronises the stream. */
RGX_API int rgx_reset_counters(rgx_ctx* ctx, rgx_stream stream);
RGX_API int rgx_read_counters(rgx_ctx* ctx, rgx_counters* out, rgx_stream stream);

/* Kernel timing for roofline reports.  While enabled, every rgx_forward /
 * rgx_backward brackets its march kernel with CUDA events on the launching stream.
 * rgx_read_kernel_times waits for the recorded events, returns the summed
 * durations (milliseconds) and launch counts since the last read, and clears them. */
RGX_API int rgx_set_profiling(rgx_ctx* ctx, int enable);
RGX_API int rgx_read_kernel_times(rgx_ctx* ctx, float* forward_ms, int* forward_launches, float* backward_ms,
                                  int* backward_launches);

/* Replaces: distCUDA2 of the reference's simple-knn submodule (submodules/simple-knn/simple_knn.cu,
 * SimpleKNN::knn; called from classes/point_cloud.py:252,592 to size the first Gaussians).
 * points [n,3] -> mean_dist2 [n]: the mean of the squared distances from each point to its three nearest
 * other points, exact (Morton sort, two levels of boxes of 32, one warp per 32 queries).  With fewer than
 * four points the missing neighbours stay at FLT_MAX in the fp32 sum, as in the reference: one missing gives
 * about FLT_MAX / 3, two or three overflow to +inf.  Needs no context; allocates
 * and frees its scratch (about 70 bytes per point) inside the call and synchronises the stream. */
RGX_API int rgx_knn_mean_dist2(int device, const float* points, int n, float* mean_dist2, rgx_stream stream);

/* Test hook (no counterpart in the reference): the workspace allocation that follows `nth` more successful
 * ones fails as if the device were out of memory, without touching the device (nth < 0 switches the hook
 * off).  After any failed allocation the call in progress returns RGX_E_CUDA, and the next call on the context
 * releases the whole workspace, so that RGX_E_NOT_BUILT is returned until rgx_build is called again. */
RGX_API int rgx_debug_fail_allocation(rgx_ctx* ctx, int nth);

/* Test hook (no counterpart in the reference): recording forwards use at most `ints` 4-byte words of the
 * recording's memory (negative: no limit), so that the rays that find no room -- which the backward then
 * searches again instead of replaying -- can be produced at will. */
RGX_API int rgx_debug_cap_recording(rgx_ctx* ctx, long long ints);

/* Two-depth lists (no counterpart in the reference).  A forward that is not followed by a backward (no
 * RGX_FLAG_SAVE_HITS, no counting) and whose view has at least `min_pairs_per_ray` (tile, Gaussian) pairs per
 * ray -- a dense scene whose rays end long before they have seen most of them -- sorts and marches only the pairs
 * that begin nearest to the eye first, about `budget_per_ray` per ray, and sorts the rest only for the tiles in
 * which some ray got further; the image is bit for bit that of the one-depth march.  Defaults 48 and 16;
 * min_pairs_per_ray < 0 switches the path off, 0 forces it; budget_per_ray = 0 keeps the current value.
 * rgx_read_two_depth returns and clears (pairs emitted, pairs sorted for the first depth, rays that went further,
 * pairs sorted for the second depth) of the latest such forward, zeros if there was none. */
RGX_API int rgx_debug_two_depth(rgx_ctx* ctx, int min_pairs_per_ray, int budget_per_ray);
RGX_API int rgx_read_two_depth(rgx_ctx* ctx, long long out[4]);

/* Lists up to a horizon for recording forwards (no counterpart in the reference).  A forward with
 * RGX_FLAG_SAVE_HITS -- a training view, whose rays end long before they have seen most of their tile's list --
 * emits, sorts and lays out only the (tile, Gaussian) pairs that begin nearest to the eye, about `budget_per_ray`
 * per ray (default 5; the horizon is picked on the device from an estimate of the pairs by distance; views with
 * fewer than 2^21 estimated pairs, or whose budget covers half of them, get complete lists).  A ray that gets as far
 * as the lists reach is marched again, on the device and before the forward's work on the stream ends, by a search
 * of the acceleration structure that needs no lists: it meets the same Gaussians in another order, so its colour is
 * that of complete lists to summation rounding (1e-5); it is not recorded, and the backward searches it again over
 * complete lists, which it then makes.  Every other ray is bit for bit what complete lists give.  No host
 * synchronisation is added: the number of such rays reaches the host behind the forward and is looked at by the next
 * call on the context; a view that had any doubles the budget for the views to come.
 * budget_per_ray = 0 switches the feature off, < 0 leaves it as it is; min_pairs >= 0 replaces the 2^21 (tests use 0
 * to take small views through it).  rgx_read_near_lists returns and clears (views whose lists stopped at a horizon,
 * the estimated number of all pairs of those views, pairs kept, views in which some ray went beyond the horizon); it
 * waits for the latest forward's count. */
RGX_API int rgx_debug_near_lists(rgx_ctx* ctx, int budget_per_ray, long long min_pairs);
RGX_API int rgx_read_near_lists(rgx_ctx* ctx, long long out[4]);

/* Per-view tile-list construction (binning + sort), timed like the march kernels while
 * profiling is enabled: summed milliseconds and number of constructions since the last
 * read, and the number of (tile, Gaussian) pairs of the latest one. */
RGX_API int rgx_read_binning(rgx_ctx* ctx, float* ms, int* runs, long long* last_pairs);

/* Measured issue-rate peaks of a device (no counterpart in the reference): fp32 FMA throughput in TFLOP/s
 * (an FMA counted as two operations) and ex2.approx throughput in 10^9 per second, with every SM busy on
 * independent register chains; a few milliseconds, synchronises.  The ceilings the march kernels (bound by
 * instruction issue, not by memory) are compared with. */
RGX_API int rgx_measure_peaks(int device, float* fma_tflops, float* ex2_gops);

/* Forward render without any allocation (no counterpart in the reference, which
 * allocates freely through cupy).  For callers that cannot call cudaMalloc when
 * they need a frame -- a viewer thread beside a trainer whose caching allocator
 * owns the device memory, a plug-in in a process that forbids allocations after
 * start-up, a latency path that cannot afford an allocation's implicit device
 * synchronisation.  (The CUDA runtime loads a kernel's code when the kernel is first launched, which may
 * allocate inside the driver: make one warm-up call during start-up, before the phase in which nothing may
 * allocate.)  Does what rgx_build + rgx_forward do (same kernels, same
 * results) with all scratch in a fixed 8 MiB array inside the library image, so it
 * needs no context and calls neither cudaMalloc nor cudaFree nor any allocating
 * library routine.  Limit: scene->n <= 32768, else RGX_E_TOO_LARGE;
 * RGX_FLAG_COUNT_WORK is rejected.  The first call on a device resolves the
 * array's device address (cudaGetSymbolAddress) and should come before any stream
 * capture.  All calls on a device share the array: calls whose GPU work overlaps
 * race; serialise them (same stream, or an event between them). */
RGX_API int rgx_forward_static(int device, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march,
                               float sigma_threshold, float* rgb, float* alpha, float* depth, rgx_stream stream);

/* How many kernels of this library the process has launched so far, over all contexts and devices (the
 * library's own kernels; the radix-sort kernels of CUB that it calls are not counted).  No counterpart in
 * the reference.  Instrumentation for benchmarks: the difference across a timed region is the number of
 * launches inside it. */
RGX_API unsigned long long rgx_kernel_launches(void);

/* Bytes of device memory currently held by the context's workspace. */
RGX_API size_t rgx_workspace_bytes(const rgx_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* RGX_H */
