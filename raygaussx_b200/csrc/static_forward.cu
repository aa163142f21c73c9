// rgx_forward_static: the forward render for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a
// frame: a viewer or capture thread running while the training process has handed
// all device memory to its framework's caching allocator, a plug-in loaded into a
// process that forbids driver allocations after start-up, or code on a latency
// path where an allocation's implicit device synchronisation is not acceptable.
// For them this file offers one entry point that does the whole forward --
// boxes, keys, sort, hierarchy refit, per-view colours, per-ray march -- with every byte
// of scratch taken from one fixed array that is part of the library image.
//
// The array is a file-scope `static __device__` object.  Its name is only a
// host-side stand-in here: host code must not pass it to a kernel.  The device
// address is obtained once per device with cudaGetSymbolAddress (with that
// device current) the first time the entry point is called on the device; that
// first call should therefore come before any stream capture.  Every GPU that
// loads the library holds the array (kScratchBytes) until the process exits.
//
// All calls on a device share the array and it keeps the last call's contents.
// Whatever has to start from a known state (reduction bounds, arrival counters of
// the refit, padding boxes) is re-initialised by the kernels of each call, on the
// caller's stream.  Two calls whose work overlaps on the GPU (different streams,
// no dependency) race on the array and give undefined images: serialise them.
#include "rgx_internal.cuh"
#include <mutex>

namespace rgx {

namespace {

constexpr int kStaticMaxGaussians = 32768;                 // stated maximum of rgx_forward_static
constexpr size_t kScratchBytes = 8u << 20;                 // 8 MiB, see the carve-up in prepare()

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {};           // device address of the array, per device
std::mutex g_setup_mutex;

struct Carver {                                             // hands out 256-byte aligned pieces of the array
    unsigned char* base;
    size_t used = 0;
    template <class T>
    T* take(size_t count) {
        size_t off = (used + 255) & ~size_t(255);
        used = off + count * sizeof(T);
        return reinterpret_cast<T*>(base + off);
    }
};

struct StaticLevels {
    int num_levels, total;
    int offset[kMaxLevels], count[kMaxLevels];
};

StaticLevels plan(int n) {                                  // same level plan as rgx_build
    StaticLevels lv{};
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

// One-time set-up for `device` (which must be current): resolve the array's device address.
int scratch_for(int device, unsigned char** out) {
    if (device < 0 || device >= kMaxDevices) return RGX_E_INVALID;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return RGX_E_CUDA;
        g_scratch_addr[device] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_addr[device];
    return RGX_OK;
}

}  // namespace

}  // namespace rgx

using namespace rgx;

extern "C" RGX_API int rgx_forward_static(int device, const rgx_scene* scene, const rgx_camera* cam,
                                          const rgx_march* march, float sigma_threshold, float* rgb, float* alpha,
                                          float* depth, rgx_stream stream) {
    if (!scene || !cam || !march || !rgb) return RGX_E_INVALID;
    const int n = scene->n;
    if (n < 0) return RGX_E_INVALID;
    if (n > kStaticMaxGaussians) return RGX_E_TOO_LARGE;     // the fixed scratch only holds this many
    const int k = scene->sh_coeffs;
    if ((k != 1 && k != 4 && k != 9 && k != 16) || scene->num_lobes < 0 || scene->num_lobes > kMaxLobes)
        return RGX_E_INVALID;
    if (n > 0 && (!scene->positions || !scene->scales || !scene->quaternions || !scene->densities ||
                  !scene->color_features))
        return RGX_E_INVALID;
    if (n > 0 && scene->num_lobes > 0 && (!scene->sg_features || !scene->sharpness || !scene->lobe_axis))
        return RGX_E_INVALID;
    // loaded 16 bytes at a time by the kernels
    if (n > 0 && (!aligned16(scene->quaternions) || (k == 16 && !aligned16(scene->color_features)))) return RGX_E_INVALID;
    if (cam->width <= 0 || cam->height <= 0 || (long long)cam->width * cam->height > (1ll << 30)) return RGX_E_INVALID;
    if (!(march->dt_step > 0.f) || march->max_prim_slice <= 0 || !(march->transmittance_eps >= 0.f) ||
        march->row_begin < 0 || march->row_end > cam->height || march->row_begin > march->row_end ||
        !(sigma_threshold > 0.f))
        return RGX_E_INVALID;
    if (march->flags & RGX_FLAG_COUNT_WORK) return RGX_E_INVALID;   // counters live in a context's workspace

    DeviceGuard guard(device);       // the caller's current device is put back on return
    if (!guard.ok) { (void)cudaGetLastError(); return RGX_E_CUDA; }
    unsigned char* base = nullptr;
    int rc = scratch_for(device, &base);
    if (rc != RGX_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;

    // carve the array up; sizes are for the maximum so that the layout never depends on the call
    const int cap = kStaticMaxGaussians;
    const StaticLevels cap_lv = plan(cap);
    Carver cv{base};
    BuildLaunch b{};
    b.keys_in = cv.take<uint64_t>(cap);  b.keys_out = cv.take<uint64_t>(cap);
    b.vals_in = cv.take<uint32_t>(cap);  b.vals_out = cv.take<uint32_t>(cap);
    b.g0 = cv.take<float4>(cap); b.g1 = cv.take<float4>(cap); b.g2 = cv.take<float4>(cap);
    b.quat = cv.take<float4>(cap); b.sdens = cv.take<float4>(cap);
    float4* rgba = cv.take<float4>(cap);
    b.hk = cv.take<float>(cap);
    b.bx = cv.take<float2>(cap_lv.total); b.by = cv.take<float2>(cap_lv.total); b.bz = cv.take<float2>(cap_lv.total);
    b.refit_counters = cv.take<unsigned int>(cap_lv.total);
    b.bounds = cv.take<int>(12);
    b.box = cv.take<SceneBox>(1);
    const size_t cub_need = build_cub_temp_bytes(cap);
    b.cub_temp = cv.take<unsigned char>(cub_need);
    b.cub_temp_bytes = cub_need;
    if (cv.used > kScratchBytes) return RGX_E_TOO_LARGE;      // would mean the constants above are inconsistent

    const int n_pad = ((n + kFan - 1) / kFan) * kFan;
    const StaticLevels lv = plan(n > 0 ? n : 1);
    Hierarchy hier{};
    hier.bx = b.bx; hier.by = b.by; hier.bz = b.bz;
    hier.num_levels = lv.num_levels;
    for (int l = 0; l < kMaxLevels; ++l) { hier.offset[l] = lv.offset[l]; hier.count[l] = lv.count[l]; }

    if (n == 0) {
        hier.count[0] = hier.count[1] = 0;
        if (cudaMemsetAsync(b.box, 0, sizeof(SceneBox), s) != cudaSuccess) return RGX_E_CUDA;
    } else {
        b.sc = *scene;
        b.sigma_threshold = sigma_threshold;
        b.morton_bits = 10;
        b.curve = RGX_CURVE_HILBERT;
        b.n_pad = n_pad;
        b.num_levels = lv.num_levels;
        for (int l = 0; l < kMaxLevels; ++l) { b.offset[l] = lv.offset[l]; b.count[l] = lv.count[l]; }
        if (launch_build(b, s) != cudaSuccess) return RGX_E_CUDA;
        ColorLaunch c{};
        c.sc = *scene;
        c.eye[0] = cam->eye[0]; c.eye[1] = cam->eye[1]; c.eye[2] = cam->eye[2];
        c.perm = b.vals_out;
        c.rgba = rgba;
        c.sigma_threshold = sigma_threshold;
        if (launch_colors(c, s) != cudaSuccess) return RGX_E_CUDA;
    }
    MarchLaunch L{};
    L.h = hier;
    L.g.g0 = b.g0; L.g.g1 = b.g1; L.g.g2 = b.g2; L.g.hk = b.hk; L.g.rgba = rgba;
    L.g.quat = b.quat; L.g.sdens = b.sdens; L.g.perm = b.vals_out;
    L.g.n = n; L.g.n_pad = n_pad;
    L.cam = *cam;
    L.m = *march;
    L.m.flags |= RGX_FLAG_PER_RAY_SEARCH;      // per-view tile lists would need a workspace sized by the view
    L.box = b.box;
    L.counters = nullptr;
    L.rgb = rgb; L.alpha = alpha; L.depth = depth;
    if (launch_march_forward(L, s) != cudaSuccess) return RGX_E_CUDA;
    return RGX_OK;
}
