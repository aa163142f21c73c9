// C ABI of librgx.so: context, workspace and the entry points of include/rgx.h.
#include "rgx_internal.cuh"
#include <atomic>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

using namespace rgx;

#ifndef RGX_BIG_GRID
#define RGX_BIG_GRID 4            // CTAs per SM of bin_emit_pairs_kernel (2, 4, 8: no difference)
#endif
// Pairs per ray that the lists of a recording forward keep.  3 M-Gaussian step: 3: rays reach the horizon, 4: 365.2 ms,
// 5: 368.6, 6: 371.9, 8: 378.6 -- what is kept has to be emitted, sorted and laid out.
#ifndef RGX_NEAR_BUDGET
#define RGX_NEAR_BUDGET 5
#endif

struct rgx_ctx {
    int device = 0;
    std::string error;
    bool alloc_failed = false;  // an allocation failed: the workspace is dropped at the next entry point
    int fail_alloc_in = -1;     // test hook: the allocation after this many more fails (rgx_debug_fail_allocation)
    long long tape_limit = -1;  // test hook: at most this many ints of the recording are used (rgx_debug_cap_recording)
    // workspace (device), grown on demand
    int cap_n_pad = 0;          // capacity in sorted slots
    int cap_boxes = 0;
    size_t cap_cub = 0;
    size_t bytes = 0;
    uint64_t *keys_in = nullptr, *keys_out = nullptr;
    uint32_t *vals_in = nullptr, *vals_out = nullptr;
    float2 *bx = nullptr, *by = nullptr, *bz = nullptr;
    float4 *g0 = nullptr, *g1 = nullptr, *g2 = nullptr, *quat = nullptr, *sdens = nullptr, *rgba = nullptr;
    float4* grad_rows = nullptr;
    bool grad_rows_clear = false;     // every row is zero (the gradient kernel clears what it reads); false after a failed backward
    unsigned char* listed = nullptr; int listed_cap = 0;   // per sorted slot: on some list of the view whose colours rgba holds
    unsigned long long listed_serial = 0;                  // the colour evaluation `listed` belongs to (0: none)
    int grad_copies = 1;     // sets of gradient rows the backward spreads its atomic additions over
    float* hk = nullptr;
    unsigned int* refit_counters = nullptr;
    unsigned char* cub_temp = nullptr;
    std::unordered_map<void*, size_t> alloc_bytes;
    int* bounds = nullptr;
    SceneBox* box = nullptr;
    DeviceCounters* counters = nullptr;
    // state of the last build
    bool built = false;
    int n = 0, n_pad = 0;
    float sigma_threshold = 0.1f;
    Hierarchy hier{};
    unsigned long long build_id = 0;   // bumped by every rgx_build
    // per-view tile lists (binning.cu)
    int bin_tiles_cap = 0;
    size_t bin_pair_cap = 0, bin_ent_cap = 0, bin_cub_cap = 0;
    uint64_t *bin_keys_in = nullptr, *bin_keys_out = nullptr;
    uint32_t *bin_vals_in = nullptr, *bin_vals_out = nullptr;
    int *tile_first = nullptr, *tile_last = nullptr, *tile_cnt = nullptr, *tile_pcnt = nullptr, *tile_pbegin = nullptr;
    int *tile_iota = nullptr, *tile_cnt_sorted = nullptr, *tile_order = nullptr;
    int* tile_unrecorded = nullptr;   // per tile: some ray of the latest recording forward could not be recorded
    int* ent_id = nullptr;
    float2 *ent_range = nullptr, *ent_blk = nullptr;
    float4* tile_dir = nullptr;
    unsigned char* bin_cub = nullptr;
    int* big_slot = nullptr;
    uint2* big_rect = nullptr;
    int big_cap = 0, sm_count = 0;
    unsigned long long* bin_total_dev = nullptr;
    unsigned long long* bin_total_host = nullptr;      // pinned
    // two-depth lists of forward-only views (binning.cu, march_lists.cu HZ variant)
    int *tile_more = nullptr, *tile_resume = nullptr; int hz_tiles_cap = 0;
    float4* hz_state = nullptr; long long hz_state_cap = 0;
    unsigned long long* hz_scalars = nullptr; unsigned long long* hz_scalars_host = nullptr;   // [0] selected pairs, [1] stopped rays (low 32 bits)
    int hz_min_pairs_per_ray = 48, hz_budget_per_ray = 16;                        // when to use them, how deep the first phase goes
    long long hz_last[4] = {0, 0, 0, 0};                                          // pairs of the view (estimate), sorted in phase 1, rays stopped, sorted in phase 2
    // what the current lists were made for
    int last_pairs = 0;
    float binning_ms = 0.f; int binning_runs = 0;
    float kept_ms[2] = {0.f, 0.f}; int kept_n[2] = {0, 0};
    bool lists_valid = false;
    // lists of a recording forward's view may hold only the pairs that begin before a horizon (lists_from_pairs)
    bool lists_partial = false;
    float lists_horizon = 0.f;
    long long lists_rays = 0;          // rays of the view the partial lists were made for
    int near_budget_per_ray = RGX_NEAR_BUDGET;   // pairs per ray such lists keep; doubled whenever a ray reached the horizon
    long long near_stats[4] = {0, 0, 0, 0};   // views with such lists, pairs of those views (estimate), pairs kept, views marched again
    // rays that went beyond the horizon in the latest march over such lists: counted on the device, finished there by a
    // per-ray search, and known to the host only later (settle_beyond)
    int* hz_rays = nullptr; long long hz_rays_cap = 0;
    unsigned long long* beyond_host = nullptr;   // pinned
    cudaEvent_t ev_beyond = nullptr;
    bool beyond_pending = false, beyond_recorded = false;
    long long beyond_kept = 0, beyond_lists_rays = 0; int beyond_budget = 0;   // of the lists that march used
    long long tape_beyond_rays = 0;              // rays of the current recording that went beyond (they are not recorded)
    long long near_min_pairs = 1ll << 21;     // views with fewer (estimated) pairs get complete lists
    double near_ratio = 2.0;                  // estimated pairs (tile rectangles) per pair kept up to the horizon, from the latest such view
    HorizonPick* near_pick = nullptr; HorizonPick* near_pick_host = nullptr;     // host copy pinned
    unsigned long long* near_hist = nullptr;
    uint2* g_rect = nullptr; unsigned int* g_code = nullptr; int* kept_slot = nullptr; int g_rect_cap = 0;
    int* tile_diff = nullptr; size_t tile_diff_cap = 0;
    unsigned long long lists_build_id = 0;
    rgx_camera lists_cam{};
    int lists_row_begin = 0, lists_row_end = 0;
    TileLists lists{};
    // tape of forward hits for the backward (RGX_FLAG_SAVE_HITS)
    int* tape = nullptr;
    long long tape_cap = 0;
    unsigned long long* tape_used = nullptr;
    unsigned long long* tape_used_host = nullptr;   // pinned; refreshed asynchronously after every recording forward
    long long* ray_head = nullptr;
    long long ray_head_cap = 0;
    bool tape_valid = false;
    unsigned long long rgba_serial = 0, tape_rgba_serial = 0;   // which evaluation of the per-view colours is in rgba / was recorded with
    unsigned long long tape_build_id = 0;
    rgx_camera tape_cam{};
    rgx_march tape_march{};            // the parameters that shape the slabs of the recording
    int tape_row_begin = 0, tape_row_end = 0;
    int* tape_tile_order = nullptr; int tape_order_cap = 0;   // order of the recording forward's CTAs, kept for the replay
    // lists of the view announced by rgx_hint_next_view, made on a stream of the context's own while the backward replays
    cudaStream_t side = nullptr;
    cudaEvent_t ev_main = nullptr, ev_lists = nullptr;
    bool lists_event_set = false;      // ev_lists marks the end of the latest work on `side`
    bool hint_set = false;
    rgx_camera hint_cam{};
    rgx_march hint_march{};
    int prefetched = 0;                // lists made ahead so far (instrumentation)
    // optional kernel timing
    bool profiling = false;
    struct Timed { cudaEvent_t a, b; int kind; };
    std::vector<Timed> timed;       // recorded, not yet read
    std::vector<Timed> spare;       // event pairs ready for reuse
};

namespace rgx {
static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace rgx

namespace {

int fail(rgx_ctx* ctx, int code, const std::string& msg) {
    if (ctx) ctx->error = msg;
    return code;
}

int cuda_fail(rgx_ctx* ctx, cudaError_t e, const char* where) {
    return fail(ctx, RGX_E_CUDA, std::string(where) + ": " + cudaGetErrorString(e));
}

template <class T>
cudaError_t regrow(rgx_ctx* ctx, T*& p, size_t count) {
    if (p) {
        cudaFree(p);
        ctx->bytes -= ctx->alloc_bytes[(void*)p];
        ctx->alloc_bytes.erase((void*)p);
    }
    p = nullptr;
    cudaError_t e = cudaErrorMemoryAllocation;
    if (ctx->fail_alloc_in == 0) ctx->fail_alloc_in = -1;                      // injected failure, nothing is allocated
    else {
        if (ctx->fail_alloc_in > 0) --ctx->fail_alloc_in;
        e = cudaMalloc((void**)&p, count * sizeof(T));
    }
    if (e == cudaSuccess) {
        ctx->bytes += count * sizeof(T);
        ctx->alloc_bytes[(void*)p] = count * sizeof(T);
    } else {
        p = nullptr;
        ctx->alloc_failed = true;       // capacities no longer describe the arrays: see release_workspace
        (void)cudaGetLastError();
    }
    return e;
}

// Frees every device array of the context and forgets what was built.  Called at the next entry point after
// an allocation failed half way through growing the workspace, so that no stale capacity can send a null or
// short array to a kernel: the caller gets RGX_E_NOT_BUILT until it calls rgx_build again.
void release_workspace(rgx_ctx* ctx) {
    cudaDeviceSynchronize();
    void** ptrs[] = {(void**)&ctx->keys_in, (void**)&ctx->keys_out, (void**)&ctx->vals_in, (void**)&ctx->vals_out,
                     (void**)&ctx->bx, (void**)&ctx->by, (void**)&ctx->bz, (void**)&ctx->g0, (void**)&ctx->g1,
                     (void**)&ctx->g2, (void**)&ctx->quat, (void**)&ctx->sdens, (void**)&ctx->rgba,
                     (void**)&ctx->grad_rows, (void**)&ctx->hk, (void**)&ctx->refit_counters, (void**)&ctx->cub_temp,
                     (void**)&ctx->bounds, (void**)&ctx->box, (void**)&ctx->counters, (void**)&ctx->bin_keys_in,
                     (void**)&ctx->bin_keys_out, (void**)&ctx->bin_vals_in, (void**)&ctx->bin_vals_out,
                     (void**)&ctx->tile_first, (void**)&ctx->tile_last, (void**)&ctx->tile_cnt, (void**)&ctx->tile_pcnt,
                     (void**)&ctx->tile_pbegin, (void**)&ctx->ent_id, (void**)&ctx->ent_range, (void**)&ctx->ent_blk,
                     (void**)&ctx->bin_cub, (void**)&ctx->bin_total_dev, (void**)&ctx->tape, (void**)&ctx->tape_used,
                     (void**)&ctx->ray_head, (void**)&ctx->tile_dir, (void**)&ctx->tile_iota,
                     (void**)&ctx->tile_cnt_sorted, (void**)&ctx->tile_order, (void**)&ctx->big_slot,
                     (void**)&ctx->big_rect, (void**)&ctx->tile_unrecorded, (void**)&ctx->tile_more, (void**)&ctx->tile_resume,
                     (void**)&ctx->hz_state, (void**)&ctx->hz_scalars, (void**)&ctx->tape_tile_order, (void**)&ctx->near_pick,
                     (void**)&ctx->near_hist, (void**)&ctx->g_rect, (void**)&ctx->g_code, (void**)&ctx->kept_slot, (void**)&ctx->tile_diff,
                     (void**)&ctx->listed, (void**)&ctx->hz_rays};
    for (void** p : ptrs) {
        if (*p) cudaFree(*p);
        *p = nullptr;
    }
    ctx->alloc_bytes.clear();
    ctx->bytes = 0;
    ctx->cap_n_pad = ctx->cap_boxes = 0;
    ctx->cap_cub = 0;
    ctx->bin_tiles_cap = 0;
    ctx->bin_pair_cap = ctx->bin_ent_cap = ctx->bin_cub_cap = 0;
    ctx->big_cap = 0;
    ctx->tape_cap = 0;
    ctx->ray_head_cap = 0;
    ctx->tape_order_cap = 0;
    ctx->lists_event_set = false;
    ctx->hint_set = false;
    ctx->hz_tiles_cap = 0; ctx->hz_state_cap = 0;
    ctx->g_rect_cap = 0; ctx->tile_diff_cap = 0; ctx->listed_cap = 0; ctx->listed_serial = 0;
    ctx->hz_rays_cap = 0; ctx->beyond_pending = false;
    ctx->grad_rows_clear = false;
    ctx->built = false;
    ctx->lists_valid = false;
    ctx->tape_valid = false;
    ctx->lists = TileLists{};
    ctx->alloc_failed = false;
}

struct Levels {
    int num_levels;
    int offset[kMaxLevels];
    int count[kMaxLevels];
    int total;   // padded boxes over all levels
};

Levels plan_levels(int n) {
    Levels lv{};
    int cnt = n, off = 0, l = 0;
    while (true) {
        lv.offset[l] = off;
        lv.count[l] = cnt;
        off += ((cnt + kFan - 1) / kFan) * kFan;
        ++l;
        if (l >= 2 && cnt <= kFan) break;
        cnt = (cnt + kFan - 1) / kFan;
        if (l == kMaxLevels) break;
    }
    lv.num_levels = l;
    lv.total = off;
    return lv;
}

int ensure_workspace(rgx_ctx* ctx, int n_pad, int boxes) {
    cudaError_t e = cudaSuccess;
    if (ctx->alloc_failed) release_workspace(ctx);
    if (!ctx->bounds) {
        if ((e = regrow(ctx, ctx->bounds, 12)) != cudaSuccess) return cuda_fail(ctx, e, "workspace");
        if ((e = regrow(ctx, ctx->box, 1)) != cudaSuccess) return cuda_fail(ctx, e, "workspace");
        if ((e = regrow(ctx, ctx->counters, 1)) != cudaSuccess) return cuda_fail(ctx, e, "workspace");
        cudaMemset(ctx->counters, 0, sizeof(DeviceCounters));
        cudaMemset(ctx->box, 0, sizeof(SceneBox));
    }
    if (n_pad > ctx->cap_n_pad) {
        size_t c = (size_t)n_pad + (size_t)n_pad / 8;   // head-room for densification
        c = ((c + 31) / 32) * 32;
#define RG(p) if ((e = regrow(ctx, ctx->p, c)) != cudaSuccess) return cuda_fail(ctx, e, "workspace " #p)
        RG(keys_in); RG(keys_out); RG(vals_in); RG(vals_out);
        RG(g0); RG(g1); RG(g2); RG(quat); RG(sdens); RG(rgba); RG(hk);
#undef RG
        // 64 bytes per Gaussian and copy, at most 2 GiB in all.  Measured on the 3M-Gaussian step: 1 copy 28.6,
        // 2 copies 34.6, 4 copies 36.5, 8 copies 36.3, 16 copies 35.7 Mrays/s (more copies: more to clear and add up)
        int copies = 4;
        while (copies > 1 && (size_t)copies * c * 64 > ((size_t)2 << 30)) copies >>= 1;
        if ((e = regrow(ctx, ctx->grad_rows, 4 * c * (size_t)copies)) != cudaSuccess) return cuda_fail(ctx, e, "workspace grad_rows");
        ctx->grad_rows_clear = false;
        ctx->grad_copies = copies;
        ctx->cap_n_pad = (int)c;
        size_t cub = build_cub_temp_bytes((int)c);
        if ((e = regrow(ctx, ctx->cub_temp, cub)) != cudaSuccess)
            return cuda_fail(ctx, e, "workspace cub");
        ctx->cap_cub = cub;
        ctx->cap_boxes = 0;
    }
    if (boxes > ctx->cap_boxes) {
        size_t c = (size_t)plan_levels(ctx->cap_n_pad).total;
        if ((size_t)boxes > c) c = boxes;
        if ((e = regrow(ctx, ctx->bx, c)) != cudaSuccess) return cuda_fail(ctx, e, "workspace boxes");
        if ((e = regrow(ctx, ctx->by, c)) != cudaSuccess) return cuda_fail(ctx, e, "workspace boxes");
        if ((e = regrow(ctx, ctx->bz, c)) != cudaSuccess) return cuda_fail(ctx, e, "workspace boxes");
        if ((e = regrow(ctx, ctx->refit_counters, c)) != cudaSuccess) return cuda_fail(ctx, e, "workspace boxes");
        ctx->cap_boxes = (int)c;
    }
    return RGX_OK;
}

// need_geometry: positions / scales / quaternions / densities are read by the call (rgx_gaussian_colors reads
// positions only).  Pointers that kernels load 16 bytes at a time must be 16-byte aligned (include/rgx.h).
int check_scene(rgx_ctx* ctx, const rgx_scene* sc, bool need_color, bool need_geometry = true) {
    if (!ctx) return RGX_E_INVALID;
    if (ctx->alloc_failed) release_workspace(ctx);      // the caller has made the context's device current
    if (!sc) return fail(ctx, RGX_E_INVALID, "scene is null");
    if (sc->n < 0) return fail(ctx, RGX_E_INVALID, "negative Gaussian count");
    if (sc->n > (1 << 30)) return fail(ctx, RGX_E_TOO_LARGE, "more than 2^30 Gaussians");
    if (sc->n > 0 && !sc->positions) return fail(ctx, RGX_E_INVALID, "null positions");
    if (need_geometry) {
        if (sc->n > 0 && (!sc->scales || !sc->quaternions || !sc->densities))
            return fail(ctx, RGX_E_INVALID, "null geometry tensor");
        if (sc->n > 0 && !aligned16(sc->quaternions))
            return fail(ctx, RGX_E_INVALID, "quaternions must be 16-byte aligned");
    }
    if (need_color) {
        int k = sc->sh_coeffs;
        if (k != 1 && k != 4 && k != 9 && k != 16) return fail(ctx, RGX_E_INVALID, "sh_coeffs must be 1, 4, 9 or 16");
        if (sc->num_lobes < 0 || sc->num_lobes > kMaxLobes) return fail(ctx, RGX_E_INVALID, "num_lobes out of range");
        if (sc->n > 0 && !sc->color_features) return fail(ctx, RGX_E_INVALID, "null color_features");
        if (sc->n > 0 && k == 16 && !aligned16(sc->color_features))
            return fail(ctx, RGX_E_INVALID, "color_features must be 16-byte aligned when sh_coeffs is 16");
        if (sc->n > 0 && sc->num_lobes > 0 && (!sc->sg_features || !sc->sharpness || !sc->lobe_axis))
            return fail(ctx, RGX_E_INVALID, "null spherical-Gaussian tensor");
    }
    return RGX_OK;
}

int check_march(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* m) {
    if (!cam || !m) return fail(ctx, RGX_E_INVALID, "camera or march parameters null");
    if (cam->width <= 0 || cam->height <= 0) return fail(ctx, RGX_E_INVALID, "empty image");
    if ((long long)cam->width * cam->height > (1ll << 30)) return fail(ctx, RGX_E_TOO_LARGE, "more than 2^30 rays");
    if (!(m->dt_step > 0.f)) return fail(ctx, RGX_E_INVALID, "dt_step must be positive");
    if (m->max_prim_slice <= 0) return fail(ctx, RGX_E_INVALID, "max_prim_slice must be positive");
    if (m->row_begin < 0 || m->row_end > cam->height || m->row_begin > m->row_end)
        return fail(ctx, RGX_E_INVALID, "row range outside the image");
    if (!(m->transmittance_eps >= 0.f)) return fail(ctx, RGX_E_INVALID, "transmittance_eps must be >= 0");
    return RGX_OK;
}

void fill_sorted(const rgx_ctx* ctx, SortedGaussians& g) {
    g.g0 = ctx->g0; g.g1 = ctx->g1; g.g2 = ctx->g2; g.hk = ctx->hk; g.rgba = ctx->rgba;
    g.quat = ctx->quat; g.sdens = ctx->sdens; g.perm = ctx->vals_out;
    g.n = ctx->n; g.n_pad = ctx->n_pad;
}

// listed_only: the current lists stop at a horizon; only the Gaussians that were emitted for them get their colours
// (the march, the replay of its recording and a search over the same lists meet no others).
int run_colors(rgx_ctx* ctx, const rgx_scene* sc, const float eye[3], cudaStream_t s, bool listed_only = false) {
    ColorLaunch c{};
    const bool listed = listed_only && ctx->lists_partial && ctx->g_code && ctx->listed && ctx->listed_cap >= ctx->n_pad;
    if (listed) {
        c.listed_rect = ctx->g_rect; c.listed_code = ctx->g_code; c.listed_cut = ctx->near_pick_host->cut;
        c.listed_out = ctx->listed;
    }
    c.sc = *sc;
    std::memcpy(c.eye, eye, sizeof(c.eye));
    c.perm = ctx->vals_out;
    c.rgba = ctx->rgba;
    c.sigma_threshold = ctx->sigma_threshold;
    ctx->rgba_serial++;
    ctx->listed_serial = listed ? ctx->rgba_serial : 0;
    cudaError_t e = launch_colors(c, s);
    return e == cudaSuccess ? RGX_OK : cuda_fail(ctx, e, "colour kernel");
}

// After a march over lists that stop at a horizon: the colours of all Gaussians, for the rays that went beyond it --
// a kernel that returns at once when `count` is zero.  The same evaluation as the one rgba holds (same eye): neither
// serial moves; every Gaussian then counts as listed.
int run_colors_if_beyond(rgx_ctx* ctx, const rgx_scene* sc, const float eye[3], const unsigned int* count, cudaStream_t s) {
    ColorLaunch c{};
    c.sc = *sc;
    std::memcpy(c.eye, eye, sizeof(c.eye));
    c.perm = ctx->vals_out;
    c.rgba = ctx->rgba;
    c.sigma_threshold = ctx->sigma_threshold;
    c.only_if = count;
    c.listed_out = ctx->listed_serial == ctx->rgba_serial ? ctx->listed : nullptr;
    cudaError_t e = launch_colors(c, s);
    return e == cudaSuccess ? RGX_OK : cuda_fail(ctx, e, "colour kernel");
}

// The number of rays that went beyond the horizon in the latest march over lists that stop at one was copied to the
// host behind that march; whoever needs it waits for the copy here (by then long done).  A view in which it is not
// zero makes the lists of the views to come twice as deep -- unless its own lists had fallen short of the budget:
// then the estimate was off, and has been corrected already.
void settle_beyond(rgx_ctx* ctx) {
    if (!ctx->beyond_pending) return;
    ctx->beyond_pending = false;
    if (cudaEventSynchronize(ctx->ev_beyond) != cudaSuccess) { (void)cudaGetLastError(); return; }
    const long long n = (long long)(*ctx->beyond_host & 0xffffffffull);
    if (ctx->beyond_recorded) ctx->tape_beyond_rays = n;
    if (n == 0) return;
    ctx->near_stats[3] += 1;
    if ((double)ctx->beyond_kept >= 0.75 * (double)ctx->beyond_budget * (double)ctx->beyond_lists_rays &&
        ctx->near_budget_per_ray == ctx->beyond_budget && ctx->near_budget_per_ray < (1 << 18))
        ctx->near_budget_per_ray *= 2;
}

struct ScopedTimer {   // brackets one kernel launch with events when profiling is on
    rgx_ctx* ctx;
    cudaStream_t s;
    rgx_ctx::Timed t{};
    bool on = false;
    ScopedTimer(rgx_ctx* c, cudaStream_t st, int kind) : ctx(c), s(st) {
        if (!c->profiling || c->timed.size() >= 65536) return;
        if (!c->spare.empty()) { t = c->spare.back(); c->spare.pop_back(); }
        else if (cudaEventCreate(&t.a) != cudaSuccess || cudaEventCreate(&t.b) != cudaSuccess) return;
        t.kind = kind;
        on = cudaEventRecord(t.a, s) == cudaSuccess;
    }
    ~ScopedTimer() {
        if (!on) return;
        cudaEventRecord(t.b, s);
        ctx->timed.push_back(t);
    }
};

// Work of the context's own stream (lists made ahead) is ordered before whatever `s` gets next.
void join_side(rgx_ctx* ctx, cudaStream_t s) {
    if (ctx->lists_event_set) cudaStreamWaitEvent(s, ctx->ev_lists, 0);
}

}  // namespace

extern "C" {

int rgx_create(int device, rgx_ctx** out) {
    if (!out) return RGX_E_INVALID;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) return RGX_E_CUDA;
    rgx_ctx* ctx = new (std::nothrow) rgx_ctx();
    if (!ctx) return RGX_E_INVALID;
    ctx->device = device;
    *out = ctx;
    return RGX_OK;
}

void rgx_destroy(rgx_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    release_workspace(ctx);
    if (ctx->bin_total_host) cudaFreeHost(ctx->bin_total_host);
    if (ctx->tape_used_host) cudaFreeHost(ctx->tape_used_host);
    if (ctx->near_pick_host) cudaFreeHost(ctx->near_pick_host);
    if (ctx->beyond_host) cudaFreeHost(ctx->beyond_host);
    if (ctx->ev_beyond) cudaEventDestroy(ctx->ev_beyond);
    if (ctx->hz_scalars_host) cudaFreeHost(ctx->hz_scalars_host);
    if (ctx->side) cudaStreamDestroy(ctx->side);
    if (ctx->ev_main) cudaEventDestroy(ctx->ev_main);
    if (ctx->ev_lists) cudaEventDestroy(ctx->ev_lists);
    for (auto* v : {&ctx->timed, &ctx->spare})
        for (auto& t : *v) { cudaEventDestroy(t.a); cudaEventDestroy(t.b); }
    delete ctx;
}

const char* rgx_last_error(const rgx_ctx* ctx) { return ctx ? ctx->error.c_str() : "null context"; }

size_t rgx_workspace_bytes(const rgx_ctx* ctx) { return ctx ? ctx->bytes : 0; }

int rgx_build(rgx_ctx* ctx, const rgx_scene* scene, float sigma_threshold, int morton_bits, int curve,
              rgx_stream stream) {
    if (!ctx) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    int rc = check_scene(ctx, scene, false);
    if (rc) return rc;
    if (morton_bits != 10 && morton_bits != 20) return fail(ctx, RGX_E_INVALID, "key_bits must be 10 or 20");
    if (curve != RGX_CURVE_MORTON && curve != RGX_CURVE_HILBERT) return fail(ctx, RGX_E_INVALID, "unknown curve");
    if (!(sigma_threshold > 0.f)) return fail(ctx, RGX_E_INVALID, "sigma_threshold must be positive");
    cudaStream_t s = (cudaStream_t)stream;
    const int n = scene->n;
    const int n_pad = ((n + kFan - 1) / kFan) * kFan;
    Levels lv = plan_levels(n > 0 ? n : 1);
    join_side(ctx, s);
    ctx->hint_set = false;
    if ((rc = ensure_workspace(ctx, n_pad > 0 ? n_pad : kFan, lv.total))) return rc;
    ctx->built = false;
    ctx->build_id++;
    ctx->n = n;
    ctx->n_pad = n_pad;
    ctx->sigma_threshold = sigma_threshold;
    ctx->hier.bx = ctx->bx; ctx->hier.by = ctx->by; ctx->hier.bz = ctx->bz;
    ctx->hier.num_levels = lv.num_levels;
    for (int l = 0; l < kMaxLevels; ++l) { ctx->hier.offset[l] = lv.offset[l]; ctx->hier.count[l] = lv.count[l]; }
    if (n == 0) {
        ctx->hier.count[0] = 0;
        ctx->hier.count[1] = 0;
        cudaError_t e = cudaMemsetAsync(ctx->box, 0, sizeof(SceneBox), s);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "build");
        ctx->built = true;
        return RGX_OK;
    }
    BuildLaunch b{};
    b.sc = *scene;
    b.sigma_threshold = sigma_threshold;
    b.morton_bits = morton_bits;
    b.curve = curve;
    b.n_pad = n_pad;
    b.keys_in = ctx->keys_in; b.keys_out = ctx->keys_out; b.vals_in = ctx->vals_in; b.vals_out = ctx->vals_out;
    b.bx = ctx->bx; b.by = ctx->by; b.bz = ctx->bz;
    b.g0 = ctx->g0; b.g1 = ctx->g1; b.g2 = ctx->g2; b.quat = ctx->quat; b.sdens = ctx->sdens; b.hk = ctx->hk;
    b.bounds = ctx->bounds; b.box = ctx->box; b.refit_counters = ctx->refit_counters;
    b.num_levels = lv.num_levels;
    for (int l = 0; l < kMaxLevels; ++l) { b.offset[l] = lv.offset[l]; b.count[l] = lv.count[l]; }
    b.cub_temp = ctx->cub_temp; b.cub_temp_bytes = ctx->cap_cub;
    cudaError_t e = launch_build(b, s);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "build");
    ctx->built = true;
    return RGX_OK;
}

// Dual basis of the camera axes (rows u*, v*, w* with u*.u = 1, u*.v = 0, ...), in double.
static bool camera_dual(const rgx_camera& c, float dual[3][3]) {
    const double u[3] = {c.u[0], c.u[1], c.u[2]}, v[3] = {c.v[0], c.v[1], c.v[2]}, w[3] = {c.w[0], c.w[1], c.w[2]};
    auto cross = [](const double* a, const double* b, double* o) {
        o[0] = a[1] * b[2] - a[2] * b[1]; o[1] = a[2] * b[0] - a[0] * b[2]; o[2] = a[0] * b[1] - a[1] * b[0];
    };
    double vw[3], wu[3], uv[3];
    cross(v, w, vw); cross(w, u, wu); cross(u, v, uv);
    const double det = u[0] * vw[0] + u[1] * vw[1] + u[2] * vw[2];
    if (!(det > 1e-12 || det < -1e-12)) return false;
    for (int k = 0; k < 3; ++k) { dual[0][k] = (float)(vw[k] / det); dual[1][k] = (float)(wu[k] / det); dual[2][k] = (float)(uv[k] / det); }
    return true;
}

static bool lists_cached(const rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* m) {
    return ctx->lists_valid && ctx->lists_build_id == ctx->build_id && ctx->lists_row_begin == m->row_begin &&
           ctx->lists_row_end == m->row_end && std::memcmp(&ctx->lists_cam, cam, sizeof(rgx_camera)) == 0;
}

#define RGB_(p, cnt) if ((e = regrow(ctx, ctx->p, (cnt))) != cudaSuccess) return cuda_fail(ctx, e, "tile-list workspace " #p)

static cudaError_t grow_pairs(rgx_ctx* ctx, size_t pairs) {
    size_t c = pairs + pairs / 4 + 1024;
    cudaError_t err;
    if ((err = regrow(ctx, ctx->bin_keys_in, c)) != cudaSuccess || (err = regrow(ctx, ctx->bin_keys_out, c)) != cudaSuccess ||
        (err = regrow(ctx, ctx->bin_vals_in, c)) != cudaSuccess || (err = regrow(ctx, ctx->bin_vals_out, c)) != cudaSuccess)
        return err;
    ctx->bin_pair_cap = c;
    return cudaSuccess;
}

// Emission of a view's (tile, Gaussian) pairs, unsorted, into ctx->bin_keys_in / bin_vals_in, in three steps so that
// a caller can put other launches between the second and the third: workspace and launch parameters ...
static int two_depth_workspace(rgx_ctx* ctx, int ntiles);

// How far an emission goes (binning.cu, culled emission): about budget_per_ray pairs per ray, unless the view has
// fewer than min_total (estimated) pairs or the cut would keep all of them (half of them, with `half`).
struct Cull {
    int budget_per_ray;
    unsigned long long min_total;
    bool half;
};

static int emit_setup(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* m, BinLaunch& b, int& ntiles, const Cull* cull = nullptr) {
    cudaError_t e = cudaSuccess;
    const int tiles_x = (cam->width + kBinTile - 1) / kBinTile;
    if (tiles_x > 65535) return fail(ctx, RGX_E_TOO_LARGE, "image wider than 65535 tiles");
    const int ty_first = m->row_begin / kBinTile, ty_last = (m->row_end - 1) / kBinTile;
    const int tiles_y = ty_last - ty_first + 1;
    ntiles = tiles_x * tiles_y;
    if (!ctx->bin_total_dev) {
        RGB_(bin_total_dev, 4);
        if (!ctx->bin_total_host && (e = cudaMallocHost((void**)&ctx->bin_total_host, 4 * sizeof(unsigned long long))) != cudaSuccess)
            return cuda_fail(ctx, e, "pinned scalar");
        if (cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, ctx->device) != cudaSuccess || ctx->sm_count <= 0)
            ctx->sm_count = 148;
    }
    if (ctx->n_pad > ctx->big_cap) {
        RGB_(big_slot, (size_t)ctx->n_pad); RGB_(big_rect, (size_t)ctx->n_pad);
        ctx->big_cap = ctx->n_pad;
    }
    if (ntiles + 1 > ctx->bin_tiles_cap) {
        size_t c = (size_t)ntiles + 1 + 64;
        RGB_(tile_first, c); RGB_(tile_last, c); RGB_(tile_cnt, c); RGB_(tile_pcnt, c); RGB_(tile_pbegin, c);
        RGB_(tile_dir, c); RGB_(tile_iota, c); RGB_(tile_cnt_sorted, c); RGB_(tile_order, c); RGB_(tile_unrecorded, c);
        ctx->bin_tiles_cap = (int)c;
        ctx->tape_valid = false;       // tile_unrecorded belongs to the recording and has just lost its contents
    }
    // first view of a context: room for eight tiles per Gaussian; a view that needs more runs the emission twice
    if (ctx->bin_pair_cap == 0 && (e = grow_pairs(ctx, (size_t)ctx->n_pad * 8)) != cudaSuccess)
        return cuda_fail(ctx, e, "tile-list workspace pairs");
    b = BinLaunch{};
    b.n = ctx->n; b.n_pad = ctx->n_pad;
    b.bx = ctx->bx; b.by = ctx->by; b.bz = ctx->bz;
    b.g0 = ctx->g0; b.g1 = ctx->g1; b.g2 = ctx->g2; b.quat = ctx->quat; b.sdens = ctx->sdens; b.hk = ctx->hk;
    b.tile_dir = ctx->tile_dir;
    b.cam = *cam;
    if (!camera_dual(*cam, b.dual)) return fail(ctx, RGX_E_INVALID, "camera axes are not linearly independent");
    b.row_begin = m->row_begin; b.row_end = m->row_end; b.tile = kBinTile;
    b.tiles_x = tiles_x; b.tiles_y = tiles_y; b.ty_first = ty_first;
    b.total_dev = ctx->bin_total_dev;
    b.big_slot = ctx->big_slot; b.big_rect = ctx->big_rect; b.big_grid = ctx->sm_count * RGX_BIG_GRID;
    if (cull && cull->budget_per_ray > 0) {
        // only the pairs that begin before a horizon are emitted (binning.cu)
        int rc = two_depth_workspace(ctx, ntiles);          // tile_more, and the counter of rays that reach the horizon
        if (rc) return rc;
        if (!ctx->near_pick) {
            RGB_(near_pick, 1); RGB_(near_hist, 2048);
            if (!ctx->near_pick_host && (e = cudaMallocHost((void**)&ctx->near_pick_host, sizeof(HorizonPick))) != cudaSuccess)
                return cuda_fail(ctx, e, "pinned horizon");
        }
        if (ctx->n_pad > ctx->g_rect_cap) {
            RGB_(g_rect, (size_t)ctx->n_pad); RGB_(g_code, (size_t)ctx->n_pad); RGB_(kept_slot, (size_t)ctx->n_pad);
            ctx->g_rect_cap = ctx->n_pad;
        }
        if (ctx->n_pad > ctx->listed_cap) {
            RGB_(listed, (size_t)ctx->n_pad);
            ctx->listed_cap = ctx->n_pad;
            ctx->listed_serial = 0;
        }
        const size_t diff = (size_t)(tiles_x + 1) * (size_t)(tiles_y + 1);
        if (diff > ctx->tile_diff_cap) {
            RGB_(tile_diff, diff + 64);
            ctx->tile_diff_cap = diff + 64;
        }
        b.pick = ctx->near_pick; b.near_hist = ctx->near_hist; b.g_rect = ctx->g_rect; b.g_code = ctx->g_code; b.kept_slot = ctx->kept_slot;
        b.tile_diff = ctx->tile_diff; b.tile_more = ctx->tile_more;
        const double rays = (double)cam->width * (double)(m->row_end - m->row_begin);
        b.near_target = (unsigned long long)((double)cull->budget_per_ray * rays * ctx->near_ratio);
        b.near_min_total = cull->min_total; b.near_half = cull->half ? 1 : 0;
    }
    return RGX_OK;
}

// ... the kernels and the copy of the pair count to the host, enqueued ...
static int emit_launch(rgx_ctx* ctx, BinLaunch& b, cudaStream_t s) {
    cudaError_t e;
    b.keys_in = ctx->bin_keys_in; b.vals_in = ctx->bin_vals_in; b.pair_cap = ctx->bin_pair_cap;
    if ((e = launch_bin_emit(b, s)) != cudaSuccess) return cuda_fail(ctx, e, "tile-list pairs");
    if ((e = cudaMemcpyAsync(ctx->bin_total_host, ctx->bin_total_dev, sizeof(unsigned long long), cudaMemcpyDeviceToHost, s)) != cudaSuccess)
        return cuda_fail(ctx, e, "tile-list pair count read-back");
    if (b.pick && (e = cudaMemcpyAsync(ctx->near_pick_host, b.pick, sizeof(HorizonPick), cudaMemcpyDeviceToHost, s)) != cudaSuccess)
        return cuda_fail(ctx, e, "horizon read-back");
    return RGX_OK;
}

// ... and the view's one host round trip: the sort needs the number of pairs.  A view whose pairs did not fit is
// emitted again into larger arrays.
static int emit_finish(rgx_ctx* ctx, BinLaunch& b, cudaStream_t s, int& total) {
    cudaError_t e;
    for (int attempt = 0;; ++attempt) {
        if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return cuda_fail(ctx, e, "tile-list pair count read-back");
        const unsigned long long total64 = ctx->bin_total_host[0];
        if (total64 > (1ull << 30)) return fail(ctx, RGX_E_TOO_LARGE, "more than 2^30 (tile, Gaussian) pairs in this view");
        total = (int)total64;
        if (total64 <= ctx->bin_pair_cap) return RGX_OK;
        if (attempt > 0) return fail(ctx, RGX_E_CUDA, "tile-list pairs did not fit twice");
        if ((e = grow_pairs(ctx, (size_t)total64)) != cudaSuccess) return cuda_fail(ctx, e, "tile-list workspace pairs");
        int rc = emit_launch(ctx, b, s);
        if (rc) return rc;
    }
}

static int emit_pairs(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* m, cudaStream_t s, BinLaunch& b, int& total,
                      int& ntiles, const Cull* cull = nullptr) {
    int rc = emit_setup(ctx, cam, m, b, ntiles, cull);
    if (rc || (rc = emit_launch(ctx, b, s))) return rc;
    return emit_finish(ctx, b, s, total);
}

// Sorts `count` pairs (keys, vals) into the per-tile lists and points ctx->lists at them.
static int fill_lists(rgx_ctx* ctx, BinLaunch& b, uint64_t* keys, uint32_t* vals, int count, int ntiles, cudaStream_t s) {
    cudaError_t e = cudaSuccess;
    const size_t ent_need = (((size_t)count + 32u * (size_t)ntiles + 31) / 32) * 32 + 32;
    if (ent_need > ctx->bin_ent_cap) {
        size_t c = ent_need + ent_need / 4;
        c = ((c + 31) / 32) * 32;
        RGB_(ent_id, c); RGB_(ent_range, c); RGB_(ent_blk, c / 32 + 1);
        ctx->bin_ent_cap = c;
    }
    const size_t cub_need = binning_cub_temp_bytes(ctx->bin_pair_cap, ntiles);
    if (cub_need > ctx->bin_cub_cap) {
        RGB_(bin_cub, cub_need);
        ctx->bin_cub_cap = cub_need;
    }
    b.keys_in = keys; b.vals_in = vals;
    b.keys_out = ctx->bin_keys_out; b.vals_out = ctx->bin_vals_out;
    b.pair_cap = ctx->bin_pair_cap;
    b.tile_first = ctx->tile_first; b.tile_last = ctx->tile_last; b.tile_cnt = ctx->tile_cnt; b.tile_pcnt = ctx->tile_pcnt;
    b.tile_pbegin = ctx->tile_pbegin;
    b.tile_iota = ctx->tile_iota; b.tile_cnt_sorted = ctx->tile_cnt_sorted; b.tile_order = ctx->tile_order;
    b.ent_id = ctx->ent_id; b.ent_range = ctx->ent_range; b.blk = ctx->ent_blk;
    b.cub_temp = ctx->bin_cub; b.cub_bytes = ctx->bin_cub_cap;
    if ((e = launch_bin_fill(b, count, s)) != cudaSuccess) return cuda_fail(ctx, e, "tile-list fill");
    ctx->lists.ent_id = ctx->ent_id; ctx->lists.ent_range = ctx->ent_range; ctx->lists.blk = ctx->ent_blk;
    ctx->lists.tile_pbegin = ctx->tile_pbegin; ctx->lists.tile_cnt = ctx->tile_cnt; ctx->lists.tile_order = ctx->tile_order;
    ctx->lists.tiles_x = b.tiles_x; ctx->lists.tiles_y = b.tiles_y; ctx->lists.ty_first = b.ty_first;
    return RGX_OK;
}

static void lists_now_valid(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* m, int total) {
    ctx->lists_cam = *cam;
    ctx->lists_row_begin = m->row_begin; ctx->lists_row_end = m->row_end;
    ctx->lists_build_id = ctx->build_id;
    ctx->lists_valid = true;
    ctx->lists_partial = false;
    ctx->last_pairs = total;
}

static int two_depth_workspace(rgx_ctx* ctx, int ntiles) {
    cudaError_t e = cudaSuccess;
    if (!ctx->hz_scalars) {
        RGB_(hz_scalars, 4);
        if (!ctx->hz_scalars_host && (e = cudaMallocHost((void**)&ctx->hz_scalars_host, 4 * sizeof(unsigned long long))) != cudaSuccess)
            return cuda_fail(ctx, e, "pinned scalars");
    }
    if (ntiles > ctx->hz_tiles_cap) {
        RGB_(tile_more, (size_t)ntiles + 64); RGB_(tile_resume, (size_t)ntiles + 64);
        ctx->hz_tiles_cap = ntiles + 64;
    }
    return RGX_OK;
}

// What a culled emission teaches about the next one: the estimate counts every tile of a Gaussian's rectangle, and
// what that is worth in pairs is learnt from view to view.
static void learn_ratio(rgx_ctx* ctx, int kept) {
    if (kept > 0) ctx->near_ratio = std::min(8.0, std::max(1.0, (double)ctx->near_pick_host->est_kept / (double)kept));
}

static Cull near_cull(const rgx_ctx* ctx) { return Cull{ctx->near_budget_per_ray, (unsigned long long)ctx->near_min_pairs, true}; }

// Turns the emitted pairs into ctx->lists.  The view of a recording forward -- a training view, whose rays end long
// before they have seen most of their tile's list (on the 3 M-Gaussian scene every ray ends within the nearest eighth
// of the pairs) -- was emitted only up to a horizon (emit_setup with near_only; binning.cu picks the horizon so that
// about near_budget_per_ray pairs per ray begin before it): such lists are marked partial, the march counts the rays
// that would have needed more (march_lists.cu, hz_phase 3), and forward_impl, should there be any, makes the complete
// lists and marches the view again.  Emission and sorting are nearly all of a view's list construction.
static int lists_from_pairs(rgx_ctx* ctx, BinLaunch& b, int total, int ntiles, const rgx_camera* cam, const rgx_march* m,
                            cudaStream_t s) {
    int rc;
    if ((rc = fill_lists(ctx, b, ctx->bin_keys_in, ctx->bin_vals_in, total, ntiles, s))) return rc;
    lists_now_valid(ctx, cam, m, total);
    if (b.pick && ctx->near_pick_host->cut != kAllBuckets) {
        const HorizonPick& pk = *ctx->near_pick_host;
        ctx->lists_partial = true;
        ctx->lists_horizon = bin_hist_bucket_end(b, (int)pk.cut);
        ctx->lists_rays = (long long)cam->width * (m->row_end - m->row_begin);
        ctx->near_stats[0] += 1; ctx->near_stats[1] += (long long)pk.est_total; ctx->near_stats[2] += total;
        learn_ratio(ctx, total);
    }
    return RGX_OK;
}

// Makes ctx->lists valid for this camera and row range (no-op if they already are).  near_only: see lists_from_pairs;
// complete lists are wanted otherwise, and cached lists that stop at a horizon are made again.
static int ensure_lists(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* m, cudaStream_t s, bool near_only = false,
                        bool near_cached_ok = false) {
    if (lists_cached(ctx, cam, m) && (!ctx->lists_partial || near_only || near_cached_ok)) return RGX_OK;
    ctx->lists_valid = false;
    if (m->row_end <= m->row_begin || ctx->n == 0) return RGX_OK;   // nothing to march
    ScopedTimer timer(ctx, s, 2);
    BinLaunch b;
    int total = 0, ntiles = 0;
    const Cull cull = near_cull(ctx);
    int rc = emit_pairs(ctx, cam, m, s, b, total, ntiles, near_only ? &cull : nullptr);
    if (rc) return rc;
    return lists_from_pairs(ctx, b, total, ntiles, cam, m, s);
}

// Lists of the announced view, made on the context's own stream while the stream of the caller replays a
// recording (which reads no lists).  begin: after the last launch on `s` that reads the current lists;
// end: after the caller has enqueued the rest of its work on `s`.  A view that would need a larger workspace for
// its tiles is left to the forward that renders it, and so is one whose lists fail to be made.
struct ListsAhead {
    bool active = false;
    BinLaunch b;
    int ntiles = 0;
};

static void lists_ahead_begin(rgx_ctx* ctx, cudaStream_t s, ListsAhead& a) {
    if (!ctx->hint_set) return;
    ctx->hint_set = false;
    const rgx_camera* cam = &ctx->hint_cam;
    const rgx_march* m = &ctx->hint_march;
    if ((m->flags & (RGX_FLAG_BRUTE_FORCE | RGX_FLAG_PER_RAY_SEARCH)) || ctx->n == 0 || m->row_end <= m->row_begin) return;
    if (lists_cached(ctx, cam, m)) return;
    const int tiles_x = (cam->width + kBinTile - 1) / kBinTile;
    const int ntiles = tiles_x * ((m->row_end - 1) / kBinTile - m->row_begin / kBinTile + 1);
    if (!ctx->bin_total_dev || ctx->bin_pair_cap == 0 || ctx->n_pad > ctx->big_cap || ntiles + 1 > ctx->bin_tiles_cap) return;
    if (!ctx->side) {
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        if (cudaStreamCreateWithPriority(&ctx->side, cudaStreamNonBlocking, hi) != cudaSuccess ||
            cudaEventCreateWithFlags(&ctx->ev_main, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ctx->ev_lists, cudaEventDisableTiming) != cudaSuccess) {
            (void)cudaGetLastError();
            if (ctx->side) cudaStreamDestroy(ctx->side);
            if (ctx->ev_main) cudaEventDestroy(ctx->ev_main);
            if (ctx->ev_lists) cudaEventDestroy(ctx->ev_lists);
            ctx->side = nullptr; ctx->ev_main = nullptr; ctx->ev_lists = nullptr;
            return;
        }
    }
    if (cudaEventRecord(ctx->ev_main, s) != cudaSuccess || cudaStreamWaitEvent(ctx->side, ctx->ev_main, 0) != cudaSuccess) return;
    ctx->lists_valid = false;                      // from here on the list arrays belong to the announced view
    const bool near_only = (m->flags & RGX_FLAG_SAVE_HITS) && !(m->flags & RGX_FLAG_COUNT_WORK);
    const Cull cull = near_cull(ctx);
    if (emit_setup(ctx, cam, m, a.b, a.ntiles, near_only ? &cull : nullptr) || emit_launch(ctx, a.b, ctx->side)) {
        cudaEventRecord(ctx->ev_lists, ctx->side);
        ctx->lists_event_set = true;
        return;
    }
    a.active = true;
}

static void lists_ahead_end(rgx_ctx* ctx, ListsAhead& a) {
    if (!a.active) return;
    int total = 0;
    {
        ScopedTimer timer(ctx, ctx->side, 2);
        if (emit_finish(ctx, a.b, ctx->side, total) == RGX_OK &&
            lists_from_pairs(ctx, a.b, total, a.ntiles, &ctx->hint_cam, &ctx->hint_march, ctx->side) == RGX_OK)
            ctx->prefetched++;
    }
    cudaEventRecord(ctx->ev_lists, ctx->side);
    ctx->lists_event_set = true;
}

// Forward-only march of a view with many more (tile, Gaussian) pairs than its rays will look at: the lists
// are made in two depths (binning.cu) and the march runs in two phases (march_lists.cu, HZ variant).
// handled = false: the view does not qualify; its complete lists have been made instead.
static int forward_two_depth(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* m, MarchLaunch& L, cudaStream_t s,
                             bool& handled) {
    handled = false;
    cudaError_t e = cudaSuccess;
    ctx->lists_valid = false;
    BinLaunch b;
    int total = 0, ntiles = 0, rc;
    const long long rays = (long long)cam->width * (m->row_end - m->row_begin);
    const long long all_rays = (long long)cam->width * cam->height;
    if (2 * all_rays > ctx->hz_state_cap) {
        RGB_(hz_state, (size_t)(2 * all_rays));
        ctx->hz_state_cap = 2 * all_rays;
    }
    // first depth: the pairs that begin nearest to the eye, about hz_budget_per_ray per ray -- or all of them, if the
    // view has fewer than hz_min_pairs_per_ray per ray or the budget covers them
    const Cull cull{ctx->hz_budget_per_ray > 0 ? ctx->hz_budget_per_ray : 1,
                    (unsigned long long)((long long)ctx->hz_min_pairs_per_ray * rays), false};
    {
        ScopedTimer timer(ctx, s, 2);
        if ((rc = emit_pairs(ctx, cam, m, s, b, total, ntiles, &cull))) return rc;
        if ((rc = fill_lists(ctx, b, ctx->bin_keys_in, ctx->bin_vals_in, total, ntiles, s))) return rc;
    }
    const HorizonPick pk = *ctx->near_pick_host;
    if (pk.cut == kAllBuckets || total == 0) {                     // one depth is enough: these are the complete lists
        lists_now_valid(ctx, cam, m, total);
        return RGX_OK;
    }
    learn_ratio(ctx, total);
    if ((e = cudaMemsetAsync(ctx->tile_resume, 0, sizeof(int) * (size_t)ntiles, s)) != cudaSuccess ||
        (e = cudaMemsetAsync(ctx->hz_scalars, 0, 4 * sizeof(unsigned long long), s)) != cudaSuccess)
        return cuda_fail(ctx, e, "two-depth workspace");
    L.lists = ctx->lists;
    L.hz_phase = 1; L.horizon = bin_hist_bucket_end(b, (int)pk.cut); L.hz_state = ctx->hz_state; L.tile_more = ctx->tile_more;
    L.tile_resume = ctx->tile_resume; L.hz_count = reinterpret_cast<unsigned int*>(ctx->hz_scalars + 1);
    {
        ScopedTimer timer(ctx, s, 0);
        e = launch_march_forward(L, s);
    }
    if (e != cudaSuccess) return cuda_fail(ctx, e, "forward march, first depth");
    if ((e = cudaMemcpyAsync(ctx->hz_scalars_host, ctx->hz_scalars, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
        (e = cudaStreamSynchronize(s)) != cudaSuccess)
        return cuda_fail(ctx, e, "first depth read-back");
    const long long stopped = (long long)(ctx->hz_scalars_host[1] & 0xffffffffull);
    int total2 = 0;
    if (stopped > 0) {
        // second depth: all pairs of the tiles in which a ray stopped
        {
            ScopedTimer timer(ctx, s, 2);
            b.pick = nullptr;
            b.tile_flag = ctx->tile_resume;
            if ((rc = emit_launch(ctx, b, s)) || (rc = emit_finish(ctx, b, s, total2))) return rc;
            if ((rc = fill_lists(ctx, b, ctx->bin_keys_in, ctx->bin_vals_in, total2, ntiles, s))) return rc;
        }
        L.lists = ctx->lists;
        L.hz_phase = 2;
        {
            ScopedTimer timer(ctx, s, 0);
            e = launch_march_forward(L, s);
        }
        if (e != cudaSuccess) return cuda_fail(ctx, e, "forward march, second depth");
    }
    ctx->hz_last[0] = (long long)pk.est_total; ctx->hz_last[1] = total; ctx->hz_last[2] = stopped; ctx->hz_last[3] = total2;
    ctx->last_pairs = total;
    handled = true;
    return RGX_OK;
}
#undef RGB_

static int prepare_march(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march,
                         MarchLaunch& L) {
    int rc = check_scene(ctx, scene, true);
    if (rc) return rc;
    if ((rc = check_march(ctx, cam, march))) return rc;
    if (!ctx->built || ctx->n != scene->n)
        return fail(ctx, RGX_E_NOT_BUILT, "rgx_build has not been called for this Gaussian set");
    L.h = ctx->hier;
    fill_sorted(ctx, L.g);
    L.cam = *cam;
    L.m = *march;
    L.box = ctx->box;
    L.counters = (march->flags & RGX_FLAG_COUNT_WORK) ? ctx->counters : nullptr;
    return RGX_OK;
}

static int forward_impl(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march, float* rgb,
                        float* alpha, float* depth, uchar4* frame, rgx_stream stream) {
    if (!ctx) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    MarchLaunch L{};
    int rc = prepare_march(ctx, scene, cam, march, L);
    if (rc) return rc;
    if (!rgb && !frame) return fail(ctx, RGX_E_INVALID, "colour output is null");
    cudaStream_t s = (cudaStream_t)stream;
    settle_beyond(ctx);
    join_side(ctx, s);
    L.rgb = rgb; L.alpha = alpha; L.depth = depth; L.frame = frame;
    const bool counting = (march->flags & RGX_FLAG_COUNT_WORK) != 0;
    bool have_colors = false;
    if (!(march->flags & (RGX_FLAG_BRUTE_FORCE | RGX_FLAG_PER_RAY_SEARCH))) {
        // a forward that nothing follows (no recording, no counting) and whose lists are yet to be made may take
        // the two-depth path, if the view turns out to have far more pairs than rays
        const bool forward_only = !(march->flags & (RGX_FLAG_SAVE_HITS | RGX_FLAG_COUNT_WORK)) && ctx->n > 0 &&
                                  march->row_end > march->row_begin && ctx->hz_min_pairs_per_ray >= 0;
        if (forward_only && !lists_cached(ctx, cam, march)) {
            bool handled = false;
            if ((rc = run_colors(ctx, scene, cam->eye, s))) return rc;
            have_colors = true;
            if ((rc = forward_two_depth(ctx, cam, march, L, s, handled))) return rc;
            if (handled) return RGX_OK;
        } else {
            const bool counts = (march->flags & RGX_FLAG_COUNT_WORK) != 0;
            const bool near_only = (march->flags & RGX_FLAG_SAVE_HITS) && !counts && ctx->near_budget_per_ray > 0;
            if ((rc = ensure_lists(ctx, cam, march, s, near_only, !counts))) return rc;
        }
        L.lists = ctx->lists;
    }
    if (!have_colors && (rc = run_colors(ctx, scene, cam->eye, s, L.lists.ent_id != nullptr && ctx->lists_partial && !counting)))
        return rc;
    // one march of the view over the lists in L.lists (a lambda: a view whose lists stop at a horizon may need a second one)
    auto march_once = [&]() -> int {
        cudaError_t e;
        const bool record = (march->flags & RGX_FLAG_SAVE_HITS) && L.lists.ent_id != nullptr && ctx->n > 0;
        if (march->flags & RGX_FLAG_SAVE_HITS) ctx->tape_valid = false;
        if (record) {
            const long long rays = (long long)cam->width * cam->height;
            const long long rows_rays = (long long)cam->width * (march->row_end - march->row_begin);
            if (!ctx->tape_used) {
                if ((e = regrow(ctx, ctx->tape_used, 4)) != cudaSuccess) return cuda_fail(ctx, e, "tape");
                if ((e = cudaMallocHost((void**)&ctx->tape_used_host, 4 * sizeof(unsigned long long))) != cudaSuccess)
                    return cuda_fail(ctx, e, "tape");
                for (int i = 0; i < 4; ++i) ctx->tape_used_host[i] = 0;
            }
            if (rays > ctx->ray_head_cap) {
                if ((e = regrow(ctx, ctx->ray_head, (size_t)rays)) != cudaSuccess) return cuda_fail(ctx, e, "tape");
                ctx->ray_head_cap = rays;
            }
            const int ntiles = L.lists.tiles_x * L.lists.tiles_y;
            if (ntiles > ctx->tape_order_cap) {
                if ((e = regrow(ctx, ctx->tape_tile_order, (size_t)ntiles + 64)) != cudaSuccess) return cuda_fail(ctx, e, "tape");
                ctx->tape_order_cap = ntiles + 64;
            }
            // room: 1024 ints per ray to begin with; what the previous recording asked for and half as much again when
            // that came close to the end (the counter keeps counting past the end), within half of the free memory
            long long want = rows_rays * 1024 + 4096;
            const long long seen = (long long)*ctx->tape_used_host;
            if (seen > (ctx->tape_cap / 8) * 7) want = want > seen + seen / 2 ? want : seen + seen / 2;
            if (want > ctx->tape_cap) {
                size_t free_b = 0, total_b = 0;
                if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
                    const long long room = (long long)((free_b + (size_t)ctx->tape_cap * sizeof(int)) / 2 / sizeof(int));
                    if (want > room) want = room;
                }
            }
            if (want > ctx->tape_cap) {
                if ((e = regrow(ctx, ctx->tape, (size_t)want)) != cudaSuccess) {
                    // no memory for a larger tape: render without one, the backward searches again
                    (void)cudaGetLastError();
                    ctx->tape = nullptr;
                    ctx->tape_cap = 0;
                    ctx->alloc_failed = false;     // nothing else depends on this array
                } else {
                    ctx->tape_cap = want;
                }
            }
            if ((e = cudaMemsetAsync(ctx->tape_used, 0, 4 * sizeof(unsigned long long), s)) != cudaSuccess ||
                (e = cudaMemsetAsync(ctx->tile_unrecorded, 0, sizeof(int) * (size_t)ntiles, s)) != cudaSuccess ||
                (e = cudaMemcpyAsync(ctx->tape_tile_order, L.lists.tile_order, sizeof(int) * (size_t)ntiles, cudaMemcpyDeviceToDevice, s)) != cudaSuccess)
                return cuda_fail(ctx, e, "tape");
            if (ctx->tape) {
                L.tape = ctx->tape; L.tape_used = ctx->tape_used; L.tape_cap = ctx->tape_cap; L.ray_head = ctx->ray_head;
                L.tile_unrecorded = ctx->tile_unrecorded;
                if (ctx->tape_limit >= 0 && ctx->tape_limit < L.tape_cap) L.tape_cap = ctx->tape_limit;
            }
        }
        const bool recorded = L.tape != nullptr;
        {
            ScopedTimer timer(ctx, s, 0);
            e = launch_march_forward(L, s);
        }
        if (e != cudaSuccess) return cuda_fail(ctx, e, "forward march");
        if (recorded) {
            cudaMemcpyAsync(ctx->tape_used_host, ctx->tape_used, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s);
            ctx->tape_valid = true;
            ctx->tape_rgba_serial = ctx->rgba_serial;
            ctx->tape_build_id = ctx->build_id;
            ctx->tape_cam = *cam;
            ctx->tape_march = *march;
            ctx->tape_row_begin = march->row_begin; ctx->tape_row_end = march->row_end;
        }
        return RGX_OK;
    };
    const bool near_lists = L.lists.ent_id != nullptr && ctx->lists_partial && !counting;
    if (!near_lists) {
        if ((rc = march_once())) return rc;
        if (L.tape) ctx->tape_beyond_rays = 0;
        return RGX_OK;
    }
    // The lists hold the pairs that begin before a horizon only.  A ray that would need more is counted, listed and
    // left unrecorded by the march; the two launches behind it -- no-ops when the count is zero -- evaluate the colours
    // of all Gaussians and finish those rays by a per-ray search of the hierarchy.  The host learns the count later.
    cudaError_t e = cudaSuccess;
    const long long all_rays = (long long)cam->width * cam->height;
    if (all_rays > ctx->hz_rays_cap) {
        if ((e = regrow(ctx, ctx->hz_rays, (size_t)all_rays)) != cudaSuccess) return cuda_fail(ctx, e, "rays beyond the horizon");
        ctx->hz_rays_cap = all_rays;
    }
    if (!ctx->beyond_host && (e = cudaMallocHost((void**)&ctx->beyond_host, sizeof(unsigned long long))) != cudaSuccess)
        return cuda_fail(ctx, e, "pinned counter");
    if (!ctx->ev_beyond && (e = cudaEventCreateWithFlags(&ctx->ev_beyond, cudaEventDisableTiming)) != cudaSuccess)
        return cuda_fail(ctx, e, "event");
    L.hz_phase = 3; L.horizon = ctx->lists_horizon; L.tile_more = ctx->tile_more;
    L.hz_count = reinterpret_cast<unsigned int*>(ctx->hz_scalars + 1);
    L.hz_rays = ctx->hz_rays;
    if ((e = cudaMemsetAsync(ctx->hz_scalars + 1, 0, sizeof(unsigned long long), s)) != cudaSuccess)
        return cuda_fail(ctx, e, "horizon counter");
    if ((rc = march_once())) return rc;
    if ((rc = run_colors_if_beyond(ctx, scene, cam->eye, L.hz_count, s))) return rc;
    if ((e = launch_march_forward_listed_rays(L, (ctx->sm_count > 0 ? ctx->sm_count : 148) * 4, s)) != cudaSuccess ||
        (e = cudaMemcpyAsync(ctx->beyond_host, ctx->hz_scalars + 1, sizeof(unsigned long long), cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
        (e = cudaEventRecord(ctx->ev_beyond, s)) != cudaSuccess)
        return cuda_fail(ctx, e, "rays beyond the horizon");
    ctx->beyond_pending = true;
    ctx->beyond_recorded = L.tape != nullptr;
    ctx->beyond_kept = ctx->last_pairs; ctx->beyond_lists_rays = ctx->lists_rays; ctx->beyond_budget = ctx->near_budget_per_ray;
    return RGX_OK;
}

int rgx_forward(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march, float* rgb,
                float* alpha, float* depth, rgx_stream stream) {
    if (ctx && !rgb) return fail(ctx, RGX_E_INVALID, "rgb output is null");
    return forward_impl(ctx, scene, cam, march, rgb, alpha, depth, nullptr, stream);
}

int rgx_forward_frame(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march,
                      unsigned char* frame_rgba8, float* depth, rgx_stream stream) {
    if (ctx && !frame_rgba8) return fail(ctx, RGX_E_INVALID, "frame buffer is null");
    if (ctx && (reinterpret_cast<uintptr_t>(frame_rgba8) & 3u)) return fail(ctx, RGX_E_INVALID, "frame buffer must be 4-byte aligned");
    return forward_impl(ctx, scene, cam, march, nullptr, nullptr, depth, reinterpret_cast<uchar4*>(frame_rgba8), stream);
}

int rgx_backward(rgx_ctx* ctx, const rgx_scene* scene, const rgx_camera* cam, const rgx_march* march,
                 const float* rgb, const float* dL_drgb, const rgx_grads* grads, rgx_stream stream) {
    if (!ctx) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    MarchLaunch L{};
    int rc = prepare_march(ctx, scene, cam, march, L);
    if (rc) return rc;
    if (!rgb || !dL_drgb || !grads) return fail(ctx, RGX_E_INVALID, "null backward argument");
    if (scene->n > 0 && (!grads->positions || !grads->scales || !grads->quaternions || !grads->densities ||
                         !grads->color_features))
        return fail(ctx, RGX_E_INVALID, "null gradient tensor");
    if (scene->n > 0 && scene->sh_coeffs == 16 && !aligned16(grads->color_features))
        return fail(ctx, RGX_E_INVALID, "the color_features gradient must be 16-byte aligned when sh_coeffs is 16");
    if (scene->n > 0 && scene->num_lobes > 0 && (!grads->sg_features || !grads->sharpness || !grads->lobe_axis))
        return fail(ctx, RGX_E_INVALID, "null spherical-Gaussian gradient tensor");
    if (scene->n == 0) return RGX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    settle_beyond(ctx);
    join_side(ctx, s);
    // a backward that replays the recording of this very view finds the forward's per-view colours still in place
    // the recording is this view's: same build, camera, rows and the march parameters that shape the slabs
    const bool tape_matches = ctx->tape_valid && ctx->tape_build_id == ctx->build_id &&
                              ctx->tape_row_begin == march->row_begin && ctx->tape_row_end == march->row_end &&
                              std::memcmp(&ctx->tape_cam, cam, sizeof(rgx_camera)) == 0 &&
                              ctx->tape_march.dt_step == march->dt_step &&
                              ctx->tape_march.dynamic_sampling == march->dynamic_sampling &&
                              ctx->tape_march.max_prim_slice == march->max_prim_slice &&
                              ctx->tape_march.transmittance_eps == march->transmittance_eps;
    const bool replays = tape_matches && !(march->flags & (RGX_FLAG_BRUTE_FORCE | RGX_FLAG_PER_RAY_SEARCH));
    if (!(replays && ctx->rgba_serial == ctx->tape_rgba_serial) && (rc = run_colors(ctx, scene, cam->eye, s))) return rc;
    // the gradient kernel of the previous backward left the rows cleared; the first backward, and one after a failure, clears them
    cudaError_t e = cudaSuccess;
    if (!ctx->grad_rows_clear &&
        (e = cudaMemsetAsync(ctx->grad_rows, 0, sizeof(float4) * 4 * (size_t)ctx->cap_n_pad * (size_t)ctx->grad_copies, s)) != cudaSuccess)   // all of it: a later build may lay the rows out differently
        return cuda_fail(ctx, e, "backward memset");
    ctx->grad_rows_clear = false;
    // the rays of a view whose lists stop at a horizon met listed Gaussians only (whichever lists this backward searches)
    const bool rows_listed = ctx->listed_serial != 0 && ctx->listed_serial == ctx->rgba_serial;
    if (!(march->flags & (RGX_FLAG_BRUTE_FORCE | RGX_FLAG_PER_RAY_SEARCH))) {
        // lists that stop at a horizon serve the backward of the view whose forward found that all its rays end
        // before the horizon; any other backward gets complete lists
        if ((rc = ensure_lists(ctx, cam, march, s, false, tape_matches && ctx->tape_beyond_rays == 0))) return rc;
        L.lists = ctx->lists;
    }
    if (L.lists.ent_id && tape_matches) {
        L.tape = ctx->tape; L.tape_used = ctx->tape_used; L.tape_cap = ctx->tape_cap; L.ray_head = ctx->ray_head;
        L.tile_unrecorded = ctx->tile_unrecorded;
        L.replay_order = ctx->tape_tile_order;
        // Slabs with few hits are worked off several at a time.  The statistics are those of the latest recording
        // whose read-back has arrived (this view's, or an earlier one's: a hint, either kernel gives the same result).
        const unsigned long long slabs = ctx->tape_used_host[1], nhits = ctx->tape_used_host[2];
        L.replay_batched = slabs == 0 || nhits < 24ull * slabs;
    }
    L.rgb_in = rgb; L.dl_drgb = dL_drgb; L.grad_rows = ctx->grad_rows; L.grad_copies = ctx->grad_copies;
    // rays without a recording first: theirs is the last launch that reads the view's lists, so the lists of an
    // announced next view can be made beside the replay and the gradient assembly
    ListsAhead ahead;
    {
        ScopedTimer timer(ctx, s, 1);
        e = launch_march_backward_search(L, s);
        if (e == cudaSuccess) {
            lists_ahead_begin(ctx, s, ahead);
            e = launch_march_backward_replay(L, s);
        }
    }
    if (e != cudaSuccess) { lists_ahead_end(ctx, ahead); return cuda_fail(ctx, e, "backward march"); }
    FinalizeLaunch f{};
    f.sc = *scene;
    f.gr = *grads;
    std::memcpy(f.eye, cam->eye, sizeof(f.eye));
    f.perm = ctx->vals_out;
    f.grad_rows = ctx->grad_rows; f.grad_copies = ctx->grad_copies; f.n_pad = ctx->n_pad;
    f.listed = rows_listed ? ctx->listed : nullptr;
    f.quat = ctx->quat; f.sdens = ctx->sdens; f.hk = ctx->hk;
    f.flags = march->flags;
    e = launch_finalize(f, s);
    ctx->grad_rows_clear = e == cudaSuccess;
    lists_ahead_end(ctx, ahead);
    return e == cudaSuccess ? RGX_OK : cuda_fail(ctx, e, "gradient finalise");
}

int rgx_hint_next_view(rgx_ctx* ctx, const rgx_camera* cam, const rgx_march* march) {
    if (!ctx) return RGX_E_INVALID;
    ctx->hint_set = false;
    if (!cam && !march) return RGX_OK;
    int rc = check_march(ctx, cam, march);
    if (rc) return rc;
    ctx->hint_cam = *cam;
    ctx->hint_march = *march;
    ctx->hint_set = true;
    return RGX_OK;
}

int rgx_lists_made_ahead(const rgx_ctx* ctx) { return ctx ? ctx->prefetched : 0; }

unsigned long long rgx_kernel_launches(void) { return rgx::g_launches.load(std::memory_order_relaxed); }

int rgx_gaussian_colors(rgx_ctx* ctx, const rgx_scene* scene, const float eye[3], float* rgb_out, rgx_stream stream) {
    if (!ctx) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    int rc = check_scene(ctx, scene, true, false);
    if (rc) return rc;
    if (!eye || (!rgb_out && scene->n > 0)) return fail(ctx, RGX_E_INVALID, "null argument");
    ColorLaunch c{};
    c.sc = *scene;
    std::memcpy(c.eye, eye, sizeof(c.eye));
    c.perm = nullptr;
    c.rgb_out = rgb_out;
    c.sigma_threshold = ctx->sigma_threshold;
    cudaError_t e = launch_colors(c, (cudaStream_t)stream);
    return e == cudaSuccess ? RGX_OK : cuda_fail(ctx, e, "colour kernel");
}

int rgx_scene_box(rgx_ctx* ctx, float bb_min[3], float bb_max[3], rgx_stream stream) {
    if (!ctx || !bb_min || !bb_max) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    if (ctx->alloc_failed) release_workspace(ctx);
    if (!ctx->built) return fail(ctx, RGX_E_NOT_BUILT, "rgx_build has not been called");
    SceneBox h;
    cudaError_t e = cudaMemcpyAsync(&h, ctx->box, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "scene box read-back");
    std::memcpy(bb_min, h.lo, sizeof(h.lo));
    std::memcpy(bb_max, h.hi, sizeof(h.hi));
    return RGX_OK;
}

int rgx_debug_fail_allocation(rgx_ctx* ctx, int nth) {
    if (!ctx) return RGX_E_INVALID;
    ctx->fail_alloc_in = nth;
    return RGX_OK;
}

int rgx_debug_two_depth(rgx_ctx* ctx, int min_pairs_per_ray, int budget_per_ray) {
    if (!ctx || budget_per_ray < 0) return RGX_E_INVALID;
    ctx->hz_min_pairs_per_ray = min_pairs_per_ray;
    if (budget_per_ray > 0) ctx->hz_budget_per_ray = budget_per_ray;
    return RGX_OK;
}

int rgx_debug_near_lists(rgx_ctx* ctx, int budget_per_ray, long long min_pairs) {
    if (!ctx) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    settle_beyond(ctx);
    if (budget_per_ray >= 0) ctx->near_budget_per_ray = budget_per_ray;
    if (min_pairs >= 0) ctx->near_min_pairs = min_pairs;
    ctx->lists_valid = false;          // lists made under the old setting are not reused
    return RGX_OK;
}

int rgx_read_near_lists(rgx_ctx* ctx, long long out[4]) {
    if (!ctx || !out) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    settle_beyond(ctx);
    for (int i = 0; i < 4; ++i) { out[i] = ctx->near_stats[i]; ctx->near_stats[i] = 0; }
    return RGX_OK;
}

int rgx_read_two_depth(rgx_ctx* ctx, long long out[4]) {
    if (!ctx || !out) return RGX_E_INVALID;
    for (int i = 0; i < 4; ++i) { out[i] = ctx->hz_last[i]; ctx->hz_last[i] = 0; }
    return RGX_OK;
}

int rgx_debug_cap_recording(rgx_ctx* ctx, long long ints) {
    if (!ctx) return RGX_E_INVALID;
    ctx->tape_limit = ints;
    return RGX_OK;
}

int rgx_set_profiling(rgx_ctx* ctx, int enable) {
    if (!ctx) return RGX_E_INVALID;
    ctx->profiling = enable != 0;
    return RGX_OK;
}

int rgx_read_kernel_times(rgx_ctx* ctx, float* forward_ms, int* forward_launches, float* backward_ms,
                          int* backward_launches) {
    if (!ctx || !forward_ms || !forward_launches || !backward_ms || !backward_launches) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    float sum[3] = {0.f, 0.f, 0.f};
    int cnt[3] = {0, 0, 0};
    for (auto& t : ctx->timed) {
        float ms = 0.f;
        if (cudaEventSynchronize(t.b) == cudaSuccess && cudaEventElapsedTime(&ms, t.a, t.b) == cudaSuccess) {
            sum[t.kind] += ms;
            cnt[t.kind] += 1;
        }
        ctx->spare.push_back(t);
    }
    ctx->timed.clear();
    sum[0] += ctx->kept_ms[0]; cnt[0] += ctx->kept_n[0]; sum[1] += ctx->kept_ms[1]; cnt[1] += ctx->kept_n[1];
    ctx->kept_ms[0] = ctx->kept_ms[1] = 0.f; ctx->kept_n[0] = ctx->kept_n[1] = 0;
    *forward_ms = sum[0]; *forward_launches = cnt[0];
    *backward_ms = sum[1]; *backward_launches = cnt[1];
    ctx->binning_ms += sum[2]; ctx->binning_runs += cnt[2];
    return RGX_OK;
}

int rgx_read_binning(rgx_ctx* ctx, float* ms, int* runs, long long* last_pairs) {
    if (!ctx || !ms || !runs || !last_pairs) return RGX_E_INVALID;
    float f, b; int nf, nb;
    int rc = rgx_read_kernel_times(ctx, &f, &nf, &b, &nb);   // drains the events; forward/backward sums are put back below
    if (rc) return rc;
    ctx->kept_ms[0] += f; ctx->kept_n[0] += nf; ctx->kept_ms[1] += b; ctx->kept_n[1] += nb;
    *ms = ctx->binning_ms; *runs = ctx->binning_runs; *last_pairs = ctx->last_pairs;
    ctx->binning_ms = 0.f; ctx->binning_runs = 0;
    return RGX_OK;
}

int rgx_reset_counters(rgx_ctx* ctx, rgx_stream stream) {
    if (!ctx) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    int rc = ensure_workspace(ctx, ctx->cap_n_pad, ctx->cap_boxes);
    if (rc) return rc;
    cudaError_t e = cudaMemsetAsync(ctx->counters, 0, sizeof(DeviceCounters), (cudaStream_t)stream);
    return e == cudaSuccess ? RGX_OK : cuda_fail(ctx, e, "counter reset");
}

int rgx_read_counters(rgx_ctx* ctx, rgx_counters* out, rgx_stream stream) {
    if (!ctx || !out) return RGX_E_INVALID;
    DeviceGuard guard(ctx->device);
    int rc = ensure_workspace(ctx, ctx->cap_n_pad, ctx->cap_boxes);
    if (rc) return rc;
    static_assert(sizeof(rgx_counters) == sizeof(DeviceCounters), "counter layouts must match");
    cudaError_t e = cudaMemcpyAsync(out, ctx->counters, sizeof(DeviceCounters), cudaMemcpyDeviceToHost,
                                    (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    return e == cudaSuccess ? RGX_OK : cuda_fail(ctx, e, "counter read-back");
}

}  // extern "C"
