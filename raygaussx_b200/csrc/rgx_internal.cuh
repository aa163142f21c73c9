// Internal declarations shared by the translation units of librgx.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <float.h>
#include "../../include/rgx.h"

namespace rgx {

constexpr int kFan = 32;          // children per hierarchy node = lanes per warp
constexpr int kMaxLevels = 8;     // level 0 = Gaussians; 32^7 > 3e10 primitives
constexpr int kSlab = 32;         // samples per slab  (BUFFER_SIZE, cuda_train/forward/gaussians_aabb.h:2)
constexpr int kChunk = 16;        // samples per chunk (CHUNK_SIZE, :3)
constexpr int kMaxLobes = 8;

// Pointers that kernels read or write 16 bytes at a time (float4) must start on a 16-byte boundary.
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Makes `device` current for the duration of an entry point and puts the caller's device back afterwards.
struct DeviceGuard {
    int prev = -1, dev;
    bool ok;
    explicit DeviceGuard(int device) : dev(device) {
        if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; (void)cudaGetLastError(); }
        ok = prev == device || cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceGuard() { if (prev >= 0 && prev != dev) cudaSetDevice(prev); }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};

// Hierarchy over the Morton-sorted Gaussians.  Level 0 holds one box per Gaussian,
// node j of level l+1 bounds boxes [32j, 32j+32) of level l.  All levels live in
// one set of arrays; every level is padded to a multiple of 32 entries with
// inverted (never hit) boxes.
struct Hierarchy {
    const float2* bx;  // per box: (min, max) along x
    const float2* by;
    const float2* bz;
    int num_levels;            // including level 0
    int offset[kMaxLevels];    // first box of each level
    int count[kMaxLevels];     // valid boxes of each level (unpadded)
};

// Per-Gaussian data in sorted order (index j), n_pad = roundup(n, 32) entries.
struct SortedGaussians {
    // g0 = (p.x, p.y, p.z, m00), g1 = (m01, m02, m10, m11), g2 = (m12, m20, m21, m22)
    // with M = S^-1 R^T / k, so that the truncation ellipsoid is |M (x - p)|^2 < 1.
    const float4* g0;
    const float4* g1;
    const float4* g2;
    const float* hk;     // log2(sigma / sigma_threshold): exp(-power/2) = exp2(-hk * |M(x-p)|^2)
    const float4* rgba;  // per view: (r*sigma, g*sigma, b*sigma, sigma)
    const float4* quat;  // raw quaternion (backward)
    const float4* sdens; // (s.x, s.y, s.z, sigma) raw (backward)
    const uint32_t* perm;// sorted index -> caller's index
    int n;
    int n_pad;
};

struct DeviceCounters {   // mirrors rgx_counters
    unsigned long long v[20];
};
enum { C_RAYS, C_SLABS, C_SLABS_HIT, C_CLOSEST, C_HITS, C_PAIRS, C_OVF, C_NODE_TESTS, C_PRIM_TESTS, C_ELL_TESTS,
       C_STACK_OVF, C_HASH, C_CANDS, C_CYC_WINDOW, C_CYC_SEEK, C_CYC_SEARCH,
       C_CYC_EVAL, C_CYC_COMP, C_CYC_WAIT, C_CYC_TOTAL, C_NUM };

struct SceneBox {         // written by the build, read by the march kernels
    float lo[3];
    float hi[3];
};

constexpr int kBinTile = 16;      // pixels per side of a binning tile

// Per-view, per-tile candidate lists (binning.cu).  Tile t owns entries
// [tile_pbegin[t], tile_pbegin[t] + roundup32(tile_cnt[t])), sorted by near distance;
// padding entries have the empty range (+inf, -inf).
struct TileLists {
    const int* ent_id;         // sorted slot of the candidate
    const float2* ent_range;   // (near, far) distance of its box from the eye, conservative
    const float2* blk;         // per 32 entries: (smallest near, largest far)
    const int* tile_pbegin;
    const int* tile_cnt;
    const int* tile_order;     // tiles by falling list length: CTA b marches tile tile_order[b] (null: tile b)
    int tiles_x, tiles_y, ty_first;
};

// Horizon of a culled emission (binning.cu): picked on the device from a histogram of the Gaussians' nearest
// distances, read by the emission kernels of the same stream and, afterwards, by the host.
struct HorizonPick {
    unsigned int cut;                   // last histogram bucket kept; kAllBuckets: every pair is kept
    unsigned int chord_bits;            // largest chord of a tile (float bits), from bin_tile_dirs_kernel
    unsigned long long est_kept;        // estimated pairs up to the cut (tile rectangles, an upper bound)
    unsigned long long est_total;       // estimated pairs of the view
    unsigned long long reserved;
};
constexpr unsigned int kAllBuckets = 0xffffffffu;

struct BinLaunch {
    int n, n_pad;
    const float2 *bx, *by, *bz;            // level-0 boxes
    const float4 *g0, *g1, *g2, *quat, *sdens;
    const float* hk;
    rgx_camera cam;
    float dual[3][3];                      // dual basis of (u, v, w): rows u*, v*, w*
    int row_begin, row_end, tile, tiles_x, tiles_y, ty_first;
    uint64_t *keys_in, *keys_out;          // [pair capacity] (tile, near distance, sorted slot)
    uint32_t *vals_in, *vals_out;          // [pair capacity] far distance (float bits)
    unsigned long long pair_cap;
    int *tile_first, *tile_last, *tile_cnt, *tile_pcnt, *tile_pbegin;   // [tiles + 1]
    int *tile_iota, *tile_cnt_sorted, *tile_order;                      // [tiles]
    int* ent_id; float2* ent_range; float2* blk;
    float4* tile_dir;                      // [tiles] central ray direction, chord to the farthest corner ray
    void* cub_temp; size_t cub_bytes;
    unsigned long long* total_dev;         // [4]; [0] = number of pairs met by the emission (may exceed pair_cap)
    int* big_slot; uint2* big_rect;        // [n_pad] complete emission: the Gaussians that touch a tile, and their tile rectangles
    int big_grid;                          // CTAs that work the list off (a few per SM)
    // culled emission (null / unused for a complete one): only the pairs that begin before a horizon are emitted
    HorizonPick* pick;
    unsigned long long* near_hist;         // [2048] estimated pairs by nearest distance of the Gaussian
    uint2* g_rect; unsigned int* g_code;   // [n_pad] tile rectangle (x = ~0: none) and histogram bucket of every Gaussian
    int* kept_slot;                        // [n_pad] the Gaussians before the cut, in no particular order; their number in total_dev[3]
    int* tile_diff;                        // [(tiles_x + 1) * (tiles_y + 1)] corners of the rectangles of culled Gaussians
    int* tile_more;                        // [tiles] the tile has pairs that were not emitted
    unsigned long long near_target;        // estimated pairs to keep
    unsigned long long near_min_total;     // views with fewer estimated pairs are emitted completely ...
    int near_half;                         // ... and so are views of which the cut would keep all (0) or half or more (1)
    const int* tile_flag;                  // null, or [tiles]: pairs of unflagged tiles are not emitted
};

struct MarchLaunch {
    Hierarchy h;
    SortedGaussians g;
    TileLists lists;
    rgx_camera cam;
    rgx_march m;
    const SceneBox* box;
    DeviceCounters* counters;
    // forward outputs / backward inputs
    float* rgb;           // [R,3]; may be null when frame is given
    float* alpha;
    float* depth;
    uchar4* frame;        // [R] 8-bit colour (cuda_gui/helpers.h:45-58), or null
    const float* rgb_in;
    const float* dl_drgb;
    // "tape": what the forward met, kept for the backward (RGX_FLAG_SAVE_HITS).  Per slab with hits a chunk
    // [tbuffer bits, hit count, next chunk offset lo, hi, sorted slots...]; ray_head[ray] = first chunk,
    // -1 = no slab with hits, -2 = not recorded (the backward searches again).
    int* tape;
    unsigned long long* tape_used;   // [3]: ints reserved, slabs recorded, hits recorded
    int replay_batched;              // backward: work several slabs of a ray off together (few hits per slab)
    long long tape_cap;
    long long* ray_head;
    int* tile_unrecorded;   // per tile (of the lists): set by the forward when a ray of the tile got ray_head = -2
    const int* replay_order;  // backward replay: tiles in the order of the recording forward's CTAs (own copy: the lists may be remade meanwhile)
    // two-depth forward (march_lists.cu, HZ variant): 0 = off, 1 = first phase (lists up to `horizon`), 2 = second
    int hz_phase;
    float horizon;
    float4* hz_state;         // [R, 2] what a ray put aside: (tbuffer, T, tenter, mode), colour and depth
    const int* tile_more;     // per tile: has pairs that begin beyond the horizon
    int* tile_resume;         // per tile: some ray stopped at the horizon
    unsigned int* hz_count;   // rays that stopped
    int* hz_rays;             // hz_phase 3: their numbers, for march_forward_listed_rays_kernel
    float4* grad_rows;    // [grad_copies, n_pad, 4] float4 of accumulated moments, layout in emit_global
    int grad_copies;      // power of two
};

struct ColorLaunch {
    rgx_scene sc;
    float eye[3];
    const uint32_t* perm;  // null: identity order, write rgb_out [n,3]
    float4* rgba;          // sorted order output (when perm != null)
    float* rgb_out;
    float sigma_threshold;
    // lists that stop at a horizon (binning.cu): the Gaussians none of whose pairs were emitted keep whatever rgba holds
    const uint2* listed_rect;
    const unsigned int* listed_code;
    unsigned int listed_cut;
    unsigned char* listed_out;   // [n_pad] 1 where the Gaussian is on some list of the view (written with listed_code)
    const unsigned int* only_if; // not null: the kernel does nothing when this counter is zero
};

struct FinalizeLaunch {
    rgx_scene sc;
    rgx_grads gr;
    float eye[3];
    const uint32_t* perm;
    float4* grad_rows;         // [grad_copies, n_pad, 4], see emit_global; the kernel leaves them cleared for the next backward
    const unsigned char* listed;   // null, or [n_pad]: the march can only have met the Gaussians marked here
    int grad_copies, n_pad;
    const float4 *quat, *sdens;   // sorted copies the march used
    const float* hk;
    int flags;
};

struct BuildLaunch {
    rgx_scene sc;
    float sigma_threshold;
    int morton_bits;
    int curve;
    int n_pad;
    // outputs
    uint64_t* keys_in; uint64_t* keys_out;
    uint32_t* vals_in; uint32_t* vals_out;
    float2 *bx, *by, *bz;
    float4 *g0, *g1, *g2, *quat, *sdens;
    float* hk;
    int* bounds;           // 12 ints: ordered-int encodings of scene box lo[3],hi[3], centre lo[3],hi[3]
    SceneBox* box;
    unsigned int* refit_counters;
    int num_levels;
    int offset[kMaxLevels];
    int count[kMaxLevels];
    void* cub_temp; size_t cub_temp_bytes;
};

// Counts the kernels of this library that were launched by this process (rgx_kernel_launches).
void note_launch();

// host launchers (each returns the cudaError_t of its last launch)
cudaError_t launch_build(const BuildLaunch& b, cudaStream_t s);
size_t build_cub_temp_bytes(int n_pad);
cudaError_t launch_colors(const ColorLaunch& c, cudaStream_t s);
cudaError_t launch_finalize(const FinalizeLaunch& f, cudaStream_t s);
size_t binning_cub_temp_bytes(size_t pair_cap, int ntiles);
cudaError_t launch_bin_emit(const BinLaunch& b, cudaStream_t s);
cudaError_t launch_bin_fill(const BinLaunch& b, int total, cudaStream_t s);
float bin_hist_bucket_end(const BinLaunch& b, int bucket);
cudaError_t launch_march_forward(const MarchLaunch& m, cudaStream_t s);
// The rays listed in m.hz_rays by a march over lists that stop at a horizon, again by per-ray search (march.cu).
cudaError_t launch_march_forward_listed_rays(const MarchLaunch& m, int ctas, cudaStream_t s);
// The backward in two launches: rays without a recording (searches the lists or the hierarchy), then the replay of
// the recording, which reads neither lists nor hierarchy.
cudaError_t launch_march_backward_search(const MarchLaunch& m, cudaStream_t s);
cudaError_t launch_march_backward_replay(const MarchLaunch& m, cudaStream_t s);

}  // namespace rgx
