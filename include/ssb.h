/*
 * ssb.h -- C ABI of libssb_b200: the per-iteration training hot path of a 3D
 * Gaussian splatting trainer (projection, tile keys, 64-bit radix sort, tile
 * ranges, tile rasteriser forward/backward, fused L1+SSIM loss, Adam), written
 * for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every pointer named d_* or documented "device" is a CUDA device pointer
 *    on the current device.  The library never allocates device memory behind
 *    the caller's back except inside an SsbStep object (ssb_step_create), and
 *    never frees caller memory.
 *  - Every function returns 0 (SSB_OK) or a negative SsbStatus.  Nothing here
 *    calls exit() or throws across the boundary; ssb_last_error_string() gives
 *    the text of the calling thread's last failure.
 *  - `stream` is a cudaStream_t passed as void*; NULL is the legacy default
 *    stream, which is where the reference launches everything
 *    (src/core/Common.cuh:207-209).
 *  - Layouts of splat parameters, gradients and optimiser moments are the
 *    reference's pool-slot layouts (src/primitives/PrimitiveBase3DGS.cuh:87-117):
 *    six arrays, each array-of-structs per splat, fp32.
 *  - Projected ("screen") splats travel between the kernels of this library as
 *    one 48-byte record per (view, splat) pair, SsbScreenRec.  ssb_screen_unpack
 *    / ssb_screen_pack convert to and from the reference's five ScreenBuffer
 *    arrays (src/primitives/PrimitiveBase3DGS.cuh:187-211).
 *
 * Each entry point names the reference interface it stands in for.
 */
#ifndef SSB_H_
#define SSB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum SsbStatus {
    SSB_OK = 0,
    SSB_ERR_INVALID_ARGUMENT = -1, /* reference: throw std::runtime_error, src/core/Common.cuh:133-146 */
    SSB_ERR_CUDA = -2,             /* reference: CHECK_DEVICE_ERROR prints and exits, src/core/Common.cuh:195-203 */
    SSB_ERR_CAPACITY = -3,         /* an output buffer sized by the caller is too small */
    SSB_ERR_OUT_OF_MEMORY = -4,    /* reference: throw_out_of_memory, src/backend/api/BackendRuntime.h:114-143 */
    SSB_ERR_UNSUPPORTED = -5,
    SSB_ERR_PEER = -6,             /* another rank did not take part in a multi-GPU step (barrier failed or timed out) */
    SSB_ERR_IO = -7                /* a checkpoint file could not be opened, read or written */
} SsbStatus;

enum { SSB_CAMERA_PINHOLE = 0, SSB_CAMERA_FISHEYE = 1, SSB_CAMERA_EQUISOLID = 2, SSB_CAMERA_EQUIRECT = 3 }; /* src/core/Common.cuh:96-101 */

enum { SSB_NUM_SH = 15, SSB_TILE = 16, SSB_SCREEN_REC_FLOATS = 12 };

/* Six per-splat arrays: parameters, their gradients, or one Adam moment.
 * Reference: _BasePrimitive3DGS::WorldBuffer, src/primitives/PrimitiveBase3DGS.cuh:87-117. */
typedef struct SsbSplats {
    float* means;        /* [n][3] */
    float* quats;        /* [n][4]  w,x,y,z, not necessarily unit */
    float* scales;       /* [n][3]  log */
    float* opacities;    /* [n]     logit */
    float* features_dc;  /* [n][3] */
    float* features_sh;  /* [n][15][3] band-major, rgb interleaved; NULL when the SH values are quantised */
} SsbSplats;

/* Quantised SH value storage, QuantizedTensor<BITS,256> (src/core/Tensor.h:1313-1404)
 * as read by the projection kernels (src/shaders/harmonics.slang:115-140). */
typedef struct SsbShQuant {
    void* packed;          /* uint8 [n*45] or uint16 [n*45]; NULL = fp32 SH */
    float* bounds;         /* float2 (min,max) per block of `bounds_stride` cells */
    int32_t bits;          /* 8 or 16 (32 / 0 = not quantised) */
    int32_t reserved;
    int64_t bounds_stride; /* cells per bound; 256 for the per-cell-block layout */
} SsbShQuant;

/* One batch of cameras sharing size and model.
 * Reference: the (viewmats, intrins, camera_model, width, height) arguments of
 * projection_3dgs_forward, src/kernels/projection/ProjectionFwd.cuh:14-78. */
typedef struct SsbCameras {
    const float* d_viewmats; /* device [count][16] row-major world-to-camera */
    const float* d_intrins;  /* device [count][4] fx, fy, cx, cy */
    int32_t count;
    int32_t width, height;
    int32_t model;           /* SSB_CAMERA_* */
    int32_t antialiased;     /* 0 = 3dgs, 1 = mip-splatting blur and opacity compensation */
    int32_t distortion;      /* SSB_DISTORTION_*: the lens-distortion tier applied to the camera model's normalised
                              * coordinates (CameraDistortionType, src/core/Common.cuh:104-109;
                              * src/shaders/projection_utils.slang:208-298).  The pairs the reference instantiates
                              * (src/kernels/projection/CameraVariants.cuh:11-22) are built: every tier for the pinhole,
                              * OpenCV and thin prism for the two fisheyes, none for the equirectangular camera; any
                              * other pair makes the projection calls return SSB_ERR_UNSUPPORTED. */
    int32_t sh_degree_plus1; /* active SH degree + 1 (the reference's sh_degree_to_use, src/app/TrainerCore.cpp:948, which picks
                              * Vanilla3DGS<0..3>): bands above it are neither read nor given a gradient.  0 = all bands of
                              * the 15-coefficient buffer (degree 3); values above 4 are refused. */
    const float* d_dist_coeffs; /* device [count][8], one row per view in the tier's own order; NULL reads as zeros.
                                 * OpenCV: k1 k2 p1 p2.  Thin prism: k1 k2 k3 k4 p1 p2 sx1 sy1.
                                 * Rational: k1 k2 k3 k4 k5 k6 p1 p2 (k4..k6 in the denominator). */
} SsbCameras;
enum { SSB_DISTORTION_NONE = 0, SSB_DISTORTION_OPENCV = 1, SSB_DISTORTION_THIN_PRISM = 2, SSB_DISTORTION_RATIONAL = 3 };

/* 48-byte projected splat.  a = {x, y, hx, hy}: centre in pixels and the half
 * extents of the alpha >= 1/255 footprint; b = {conic a, b, c, opacity};
 * c = {r, g, b, ray depth}. */
typedef struct SsbScreenRec { float a[4], b[4], c[4]; } SsbScreenRec;

const char* ssb_last_error_string(void);

/* Kernels of this library never follow an index out of the buffers they were given.  When one meets
 * such an index (a tile range or list entry beyond the list's capacity, a record index beyond the
 * record array) it skips the entry and sets a bit in a sticky per-device status word; when the tile
 * intersection finds more pairs than the caller's buffers hold it drops the excess, clamps every
 * range it hands on and sets another.  ssb_device_status copies the word of the current device to
 * *h_bits (may be NULL), clears it, synchronises the stream and returns SSB_ERR_INVALID_ARGUMENT
 * (bad index), SSB_ERR_CAPACITY (pairs dropped) or SSB_OK.  The reference has no counterpart: it
 * sizes its buffers from the pair count read back to the host (src/kernels/tile/IntersectTile.cu:432-459). */
enum { SSB_STATUS_BAD_INDEX = 1, SSB_STATUS_PAIRS_DROPPED = 2 };
int ssb_device_status(int32_t* h_bits, void* stream);
/* "major.minor" of the ABI and the compute capability the kernels were built for. */
const char* ssb_version_string(void);

/* ---- projection --------------------------------------------------------- */

/* Replaces projection_3dgs_forward (src/kernels/projection/ProjectionFwd.cu:104-139,
 * kernel src/kernels/projection/ProjectionFwd_kernel.cuh:15-111).
 * d_aabb [C*n][4] xyxy pixels (all zero = culled), d_depths [C*n] sorting depth,
 * d_radii [n] running max over views (caller zeroes once per step; may be NULL),
 * d_screen [C*n] records (only written where the pair is kept). */
int ssb_project_fwd(const SsbSplats* splats, const SsbShQuant* shq, int64_t n,
                    const SsbCameras* cams,
                    float* d_aabb, float* d_depths, float* d_radii, SsbScreenRec* d_screen,
                    void* stream);

/* Replaces projection_3dgs_packed_forward (src/kernels/projection/ProjectionPackedFwd.cu:64-158): the
 * same projection, but only the visible (view, splat) pairs are returned, compacted in (view-major,
 * splat-minor) order, with d_camera_ids[v] / d_gaussian_ids[v] naming the view and splat of packed
 * pair v.  The pair count V goes to *d_n_visible (and, if h_n_visible is given, to the host after a
 * stream synchronisation, as the reference reads it back).  Outputs hold `capacity` pairs; pairs beyond
 * it are dropped and reported (SSB_ERR_CAPACITY when the host count is requested).  The packed arrays
 * feed ssb_intersect_tiles_packed and, through its flatten ids, the rasterisers unchanged.
 * Like the reference, two passes with a scan in between, so memory is proportional to the visible pairs: a visibility
 * pass that reads no SH and leaves one 4-byte flag per pair, an in-place scan, and a pass that projects the kept pairs
 * straight into their slots.  Workspace: ssb_project_fwd_packed_workspace_bytes(n, views), about 4 bytes per pair. */
int64_t ssb_project_fwd_packed_workspace_bytes(int64_t n, int32_t n_views);
int ssb_project_fwd_packed(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams,
                           void* d_workspace, int64_t workspace_bytes,
                           float* d_aabb, float* d_depths, float* d_radii, SsbScreenRec* d_screen,
                           int32_t* d_camera_ids, int32_t* d_gaussian_ids, int64_t capacity,
                           int64_t* d_n_visible, int64_t* h_n_visible, void* stream);

/* The packed form of ssb_project_bwd (the `packed` mode of projection_fused_bwd_kernel with its camera_ids /
 * gaussian_ids arguments, src/kernels/projection/ProjectionBwd_kernel.cuh:16-54):
 * aabb and screen-space gradients are given per packed pair with their view and splat ids; the number of
 * pairs is read from *d_n_pairs on the device (at most max_pairs).  The workspace receives the inverse map (slot of
 * every (view, splat) pair, 4 bytes each) and the per-splat kernel of ssb_project_bwd sums each splat's views through it
 * (no atomics), so the result equals the unpacked call's.
 * Workspace: ssb_project_bwd_packed_workspace_bytes(n, views), 4 bytes per pair. */
int64_t ssb_project_bwd_packed_workspace_bytes(int64_t n, int32_t n_views);
int ssb_project_bwd_packed(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams,
                           const float* d_aabb, const SsbScreenRec* d_v_screen, const int32_t* d_camera_ids, const int32_t* d_gaussian_ids,
                           const int64_t* d_n_pairs, int64_t max_pairs, void* d_workspace, int64_t workspace_bytes,
                           const SsbSplats* grads, int accumulate, void* stream);

/* Replaces projection_3dgs_backward (src/kernels/projection/ProjectionBwd.cu:134,
 * kernel src/kernels/projection/ProjectionBwd_kernel.cuh:16-130): vjp of the
 * projection and of SH-to-colour for every kept pair, summed over the views of
 * `cams`.  d_v_screen [C*n] holds gradient records laid out like SsbScreenRec
 * (a = {v_x, v_y, 0, 0}, b = {v_conic a,b,c, v_opacity}, c = {v_r, v_g, v_b, v_depth}).
 * accumulate != 0 adds to `grads`; 0 overwrites them (so no separate zeroing
 * pass is needed before the first view of a step). */
int ssb_project_bwd(const SsbSplats* splats, const SsbShQuant* shq, int64_t n,
                    const SsbCameras* cams, const float* d_aabb,
                    const SsbScreenRec* d_v_screen,
                    const SsbSplats* grads, int accumulate, void* stream);

/* Record <-> reference ScreenBuffer arrays (xy [m][2], depth [m], conic [m][3],
 * opac [m], rgb [m][3]); src/primitives/PrimitiveBase3DGS.cuh:187-211. */
int ssb_screen_unpack(const SsbScreenRec* d_screen, int64_t m,
                      float* d_xy, float* d_depth, float* d_conic, float* d_opac, float* d_rgb, void* stream);
int ssb_screen_pack(const float* d_xy, const float* d_depth, const float* d_conic, const float* d_opac,
                    const float* d_rgb, int64_t m, SsbScreenRec* d_screen, void* stream);
/* ssb_screen_unpack that ADDS the records' fields to the arrays: gradient records (the layout of ssb_project_bwd's
 * d_v_screen) onto the reference's running v_ScreenBuffer arrays, which its rasteriser backward accumulates into
 * (src/kernels/raster/RasterizationBwd.cu:142-145).  Any array may be NULL. */
int ssb_screen_unpack_add(const SsbScreenRec* d_records, int64_t m,
                          float* d_xy, float* d_depth, float* d_conic, float* d_opac, float* d_rgb, void* stream);

/* ---- tile intersection: keys, sort, ranges ------------------------------ */

/* Bytes of scratch ssb_tile_keys needs for `total` = C*n pairs. */
int64_t ssb_tile_keys_workspace_bytes(int64_t total);

/* Replaces passes 1-2 of do_intersect_tile_generic, ellipse mode, no live-tile
 * map (src/kernels/tile/IntersectTile.cu:372-479): per-pair tile counts, their
 * inclusive sum, then keys (tile_id << 32 | depth bits) and flatten ids.
 * d_tiles_per_splat / d_cum_tiles [total] (int32) may be NULL if the caller does
 * not want them.  d_n_isects (device int64) receives the pair count M; when
 * h_n_isects != NULL the call also synchronises the stream and stores M there.
 * Keys beyond `capacity` are not written and the call (when it synchronises) or
 * ssb_sort_pairs_u64 reports SSB_ERR_CAPACITY. */
int ssb_tile_keys(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                  int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                  void* d_workspace, int64_t workspace_bytes,
                  int32_t* d_tiles_per_splat, int32_t* d_cum_tiles,
                  int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                  int64_t* d_n_isects, int64_t* h_n_isects, void* stream);

int64_t ssb_sort_workspace_bytes(int64_t capacity);

/* Replaces backend::sort_pairs<int64,int32> / cub::DeviceRadixSort::SortPairs
 * (src/backend/common/SortScan.h:53-56, src/kernels/tile/IntersectTile.cu:487-497):
 * stable ascending sort on key bits [begin_bit, end_bit).  The element count is
 * read on the device from *d_n (clamped to capacity; capacity < 2^30).  *selector (host) tells
 * which buffer pair holds the result: 0 = (keys_a, vals_a), 1 = (keys_b, vals_b). */
int ssb_sort_pairs_u64(int64_t* d_keys_a, int32_t* d_vals_a, int64_t* d_keys_b, int32_t* d_vals_b,
                       const int64_t* d_n, int64_t capacity, int32_t begin_bit, int32_t end_bit,
                       void* d_workspace, int64_t workspace_bytes, int32_t* selector, void* stream);

/* Reports SSB_ERR_CUDA if a tile of the last sort that used this workspace gave
 * up waiting for its predecessor (every device-side wait in the sort is bounded;
 * the output is then not sorted).  Synchronises the stream.  d_workspace == NULL
 * names the built-in scratch of ssb_sort_pairs_u64_noalloc on the current device.
 * No reference counterpart: cub's sort has no such status. */
int ssb_sort_check(const void* d_workspace, void* stream);

/* The same sort with NO workspace argument and no allocation anywhere: its scratch
 * (look-back descriptors and digit histograms, about 1 MB) is a fixed array inside
 * the library image, present on every GPU that loads the library until the process
 * exits.  It has no counterpart in the reference (cub's sort always takes caller
 * temp storage).  Meant for callers that must not create device memory where they
 * sort: plug-ins whose host forbids cudaMalloc, or loops where an allocation's
 * device-wide synchronisation would stall other streams.
 *  - capacity may be at most 2^20 = 1,048,576 pairs; larger requests return
 *    SSB_ERR_CAPACITY and touch nothing (a negative one, SSB_ERR_INVALID_ARGUMENT).
 *  - Whether a bounded wait inside the sort gave up (the output is then unsorted) is
 *    read with ssb_sort_check(NULL, stream): the caller holds no workspace pointer to
 *    pass, so NULL stands for the built-in array of the current device.
 *  - The first call on each device looks up the array's device address (with that
 *    device current); make that first call before starting any stream capture.
 *  - All calls on a device share the one array, whose contents survive from call
 *    to call; each call re-initialises what it needs, so back-to-back calls on one
 *    stream are fine, but two calls that can run on the GPU at the same time (on
 *    different streams) race on it and corrupt each other's result. */
int ssb_sort_pairs_u64_noalloc(int64_t* d_keys_a, int32_t* d_vals_a, int64_t* d_keys_b, int32_t* d_vals_b,
                               const int64_t* d_n, int64_t capacity, int32_t begin_bit, int32_t end_bit,
                               int32_t* selector, void* stream);

/* Number of key bits the tile id occupies: smallest b with 2^b > n_tiles
 * (src/kernels/tile/IntersectTile.cu:489-490). */
int32_t ssb_tile_n_bits(int64_t n_tiles);

/* The whole of do_intersect_tile_generic (src/kernels/tile/IntersectTile.cu:372-509) in one call: the
 * sorted pair indices (flatten ids), optionally the sorted keys, the per-tile ranges and the pair
 * count, identical to ssb_tile_keys -> ssb_sort_pairs_u64 -> ssb_tile_ranges on the same inputs, but
 * built without a global sort: pairs are binned by tile (count, scan, scatter) and each tile's list
 * is sorted on (depth bits, pair index) by one CTA.  total must be a whole number of images of
 * n_per_image pairs.  d_isect_ids may be NULL when the sorted keys are not needed.  d_tile_offsets
 * receives n_images * tiles entries (range end of the last tile = *d_n_isects, as for
 * ssb_tile_ranges).  Pairs beyond capacity are dropped: *d_n_isects still reports the full count, but every
 * entry of d_tile_offsets is clamped to capacity, so the lists that lie below it are complete, the list that
 * straddles it is cut, and later tiles are empty (SSB_STATUS_PAIRS_DROPPED is raised, see ssb_device_status).
 * Workspace: ssb_intersect_tiles_workspace_bytes(n_images * tiles, capacity). */
int64_t ssb_intersect_tiles_workspace_bytes(int64_t n_tiles_total, int64_t capacity);
int ssb_intersect_tiles(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                        int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                        void* d_workspace, int64_t workspace_bytes,
                        int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                        int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream);

/* ssb_intersect_tiles for packed pairs (the packed branch of do_intersect_tile_generic): the image of
 * pair v is d_camera_ids[v], the number of pairs is read from *d_n_pairs on the device (at most
 * max_pairs), and the flatten ids written are packed pair indices.  Workspace as for
 * ssb_intersect_tiles with n_images * tiles. */
int ssb_intersect_tiles_packed(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen, const int32_t* d_camera_ids,
                               const int64_t* d_n_pairs, int64_t max_pairs, int32_t n_images, int32_t width, int32_t height,
                               void* d_workspace, int64_t workspace_bytes, int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                               int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream);

/* ---- live-tile map ------------------------------------------------------
 * Replaces compute_tile_active / tile_active_kernel (src/kernels/tile/IntersectTile.cu:309-367; caller
 * src/engine/EngineTrainStep.cpp:84-126).  d_mask [n_images][mask_h][mask_w] bytes (!= 0 = the pixel takes part in the
 * loss), nearest-sampled when its size is not the image's.  d_tile_active [n_images][tile_h][tile_w] int32 gets 1 for a
 * tile with at least one such pixel in its 16 x 16 block grown by one pixel on every side, else 0.
 * The *_live forms of the intersection calls take that map (NULL: every tile is live) as the `tile_active` argument of
 * do_intersect_tile_generic (src/kernels/tile/IntersectTile.cu:376-388): a tile marked 0 gets no pair in either pass,
 * so the pair count, the keys and the per-tile ranges are those of the live tiles and the rasterisers find an empty
 * range there. */
int ssb_tile_active(const uint8_t* d_mask, int32_t n_images, int32_t mask_h, int32_t mask_w, int32_t width, int32_t height,
                    int32_t* d_tile_active, void* stream);
int ssb_tile_keys_live(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                       int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                       void* d_workspace, int64_t workspace_bytes,
                       int32_t* d_tiles_per_splat, int32_t* d_cum_tiles,
                       int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                       int64_t* d_n_isects, int64_t* h_n_isects, const int32_t* d_tile_active, void* stream);
int ssb_intersect_tiles_live(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                             int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                             void* d_workspace, int64_t workspace_bytes,
                             int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                             int32_t* d_tile_offsets, int64_t* d_n_isects, const int32_t* d_tile_active, void* stream);
int ssb_intersect_tiles_packed_live(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen, const int32_t* d_camera_ids,
                                    const int64_t* d_n_pairs, int64_t max_pairs, int32_t n_images, int32_t width, int32_t height,
                                    void* d_workspace, int64_t workspace_bytes, int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                                    int32_t* d_tile_offsets, int64_t* d_n_isects, const int32_t* d_tile_active, void* stream);

/* Replaces intersect_offset_kernel (src/kernels/tile/IntersectTile.cu:271-307).
 * d_offsets [n_tiles_total] int32: first sorted index of each tile; tiles after
 * the last key get M; all zero when M == 0. */
int ssb_tile_ranges(const int64_t* d_sorted_ids, const int64_t* d_n, int64_t capacity,
                    int64_t n_tiles_total, int32_t* d_offsets, void* stream);

/* ---- rasteriser --------------------------------------------------------- */

/* Replaces rasterize_to_pixels_3dgs_fwd (src/kernels/raster/RasterizationFwd.cu:147-185,
 * kernel src/kernels/raster/RasterizationEval3DFwd_kernel.cuh:48-313, 2D variant).
 * Outputs: d_rgb [I][H][W][3], d_depth [I][H][W], d_T [I][H][W], d_last_ids [I][H][W].
 * d_depth may be NULL when the depth image is not needed (its accumulation is then compiled out).
 * n_records = entries of d_screen, n_flatten = entries of d_flatten_ids (the reference's tensors carry
 * their sizes; here they bound every access): tile ranges are clamped to min(*d_n_isects, n_flatten) and a
 * list entry that is not a record index below n_records is skipped and reported (ssb_device_status). */
int ssb_raster_fwd(const SsbScreenRec* d_screen, int64_t n_records, const int32_t* d_tile_offsets,
                   const int32_t* d_flatten_ids, int64_t n_flatten,
                   const int64_t* d_n_isects, int32_t n_images, int32_t width, int32_t height,
                   float* d_rgb, float* d_depth, float* d_T, int32_t* d_last_ids, void* stream);

/* Replaces rasterize_to_pixels_3dgs_bwd (src/kernels/raster/RasterizationBwd.cu:253-291,
 * kernel src/kernels/raster/RasterizationEval3DBwd_kernel.cuh:48-636, 2D variant).
 * d_v_depth and d_v_T may be NULL (treated as zero; without d_v_depth the depth channel is compiled
 * out and d_render_depth may be NULL too).  Gradients are ADDED into
 * d_v_screen [n_records] (layout as in ssb_project_bwd); the caller zeroes it.
 * n_records and n_flatten bound every access as in ssb_raster_fwd; d_last_ids entries are clamped too. */
int ssb_raster_bwd(const SsbScreenRec* d_screen, int64_t n_records, const int32_t* d_tile_offsets,
                   const int32_t* d_flatten_ids, int64_t n_flatten,
                   const int64_t* d_n_isects, int32_t n_images, int32_t width, int32_t height,
                   const float* d_render_depth, const float* d_T, const int32_t* d_last_ids,
                   const float* d_v_rgb, const float* d_v_depth, const float* d_v_T,
                   SsbScreenRec* d_v_screen, void* stream);

/* DensifyAccumMode of the reference (src/primitives/Primitive.cuh:37-39). */
enum { SSB_ACCUM_NONE = 0, SSB_ACCUM_MAX = 1, SSB_ACCUM_SUM = 2, SSB_ACCUM_AVG = 3 };

/* ssb_raster_bwd that also accumulates the per-splat densification weight
 * (accum_weight_map_buffer / o_accum_weight / o_accum_weight_den of rasterize_to_pixels_bwd_kernel,
 * src/kernels/raster/RasterizationEval3DBwd_kernel.cuh:91-101,541-550,566-579): over every fragment
 * that receives a gradient, the maximum (MAX) or the sum (SUM, AVG) of
 * d_weight_map[pixel] * alpha * T, and for AVG also the sum of alpha * T into d_accum_weight_den.
 * d_weight_map is [n_images][height][width] (NULL = all zero).  The results are combined into
 * d_accum_weight[splat] (atomic max / add; the caller zeroes it), where splat = d_gaussian_ids[record]
 * (packed projection) or record index % n_per_image when d_gaussian_ids is NULL.
 * accum_mode = SSB_ACCUM_NONE is ssb_raster_bwd. */
int ssb_raster_bwd_accum(const SsbScreenRec* d_screen, int64_t n_records, const int32_t* d_tile_offsets,
                         const int32_t* d_flatten_ids, int64_t n_flatten,
                         const int64_t* d_n_isects, int32_t n_images, int32_t width, int32_t height,
                         const float* d_render_depth, const float* d_T, const int32_t* d_last_ids,
                         const float* d_v_rgb, const float* d_v_depth, const float* d_v_T, SsbScreenRec* d_v_screen,
                         int32_t accum_mode, const float* d_weight_map, int64_t n_per_image, const int32_t* d_gaussian_ids,
                         float* d_accum_weight, float* d_accum_weight_den, void* stream);

/* ---- loss --------------------------------------------------------------- */

/* Replaces compute_multi_scale_per_pixel_losses at one scale with only the RGB
 * L1 weight set (src/kernels/loss/PerPixelLoss.cu:948-1402) followed by
 * fused_ssim_inplace_async (src/kernels/loss/FusedSSIM.cu:1211-1234, kernel :639-1022):
 * loss = w_l1 * mean|render - gt| + w_ssim * (1 - SSIM).  Writes d(loss)/d(render)
 * to d_v_render [B][H][W][3] and {L1, SSIM, loss} sums to d_losses[3] (device,
 * fp32; caller reads them whenever it likes -- the reference reads its scalars
 * one step late, src/kernels/loss/PerPixelLoss.cu:1374-1400). */
int ssb_loss_l1_ssim_fwdbwd(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                            float w_l1, float w_ssim, float* d_v_render, float* d_losses, void* stream);

/* The same with the per-pixel SSIM loss map of the densification strategy (ssim_loss_map / ssim_loss_map_weight /
 * ssim_loss_map_mode of fused_ssim_inplace_async, src/kernels/loss/FusedSSIM.cu:1211-1234; kernel :861-886,1009-1016):
 * d_loss_map[image][y][x] += weight * (1 - mean over the channels of v), v = SSIM (mode 1, SsimFull), its
 * contrast-structure factor (2, SsimCs) or its structure term (3, SsimStr); SsimLossMapMode,
 * src/kernels/loss/PerPixelLoss.cuh:129-134.  Mode 0 writes no map.  The map is what
 * ssb_raster_bwd_accum takes as d_weight_map. */
int ssb_loss_l1_ssim_fwdbwd_map(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                                float w_l1, float w_ssim, float* d_v_render, float* d_losses,
                                int32_t ssim_loss_map_mode, float ssim_loss_map_weight, float* d_loss_map, void* stream);

/* Multi-scale loss with an optional mask and the densification loss map: the colour part of
 * compute_multi_scale_per_pixel_losses (src/kernels/loss/PerPixelLoss.cu:941-1363) with fused_ssim_inplace's mask
 * handling (src/kernels/loss/FusedSSIM.cu:105-195,717-724,829-915,988-994).
 *   num_scales 1..4: level s is level s-1 pooled 2x2 (size max(1, n / 2)); every level computes
 *     w_l1 * L1 + w_ssim * (1 - SSIM) and its gradient, and the levels are averaged:
 *     d_v_render = (v_0 + sum_s 0.25^s * v_s[y >> s][x >> s]) / num_scales.
 *   d_mask [n_images][mask_h][mask_w] bytes (NULL: none), != 0 = the pixel takes part.  A mask of another size than
 *     the image is nearest-sampled.  Masked pixels leave the L1 sum (which is divided by the number of unmasked
 *     pixels) and every SSIM window, a window centred on one scores 1, and they receive no gradient.  With a mask of
 *     the image's size the pyramid pools over the unmasked children only.
 *   loss_map_mode (DensifyLossMapMode, src/kernels/loss/PerPixelLoss.cuh:98-110): 0 none; 1 the pixel's weighted L1
 *     term + w_ssim * (1 - SSIM); 2, 3, 4 w_ssim * (1 - SSIM / contrast-structure / structure).  d_loss_map
 *     [n_images][H][W] is OVERWRITTEN with the mean over the levels.  Modes 5..10 (edge-aware maps, non-maximum
 *     suppression) return SSB_ERR_UNSUPPORTED.
 * d_losses[3] (overwritten): mean over the levels of the L1 term, level 0's SSIM, mean over the levels of the total.
 * The workspace holds the pyramid (about 0.42 of the three level-0 images for 4 levels) and is sized by
 * ssb_loss_workspace_bytes for the same arguments; SSB_ERR_CAPACITY when it is too small. */
typedef struct SsbLossConfig {
    float w_l1, w_ssim;
    int32_t num_scales;
    int32_t loss_map_mode;
    const uint8_t* d_mask;
    int32_t mask_h, mask_w;
} SsbLossConfig;
int64_t ssb_loss_workspace_bytes(int32_t n_images, int32_t height, int32_t width, const SsbLossConfig* cfg);
int ssb_loss_multi_scale(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                         const SsbLossConfig* cfg, float* d_v_render, float* d_losses, float* d_loss_map, void* d_workspace,
                         int64_t workspace_bytes, void* stream);

/* ---- optimiser ---------------------------------------------------------- */

typedef struct SsbAdamConfig {
    float lr_means, lr_quats, lr_scales, lr_opacities, lr_features_dc, lr_features_sh;
    float sh_reg_weight;   /* l2_reg of fused_adam_step for DC (offset 0.5/0.2820948) and SH (offset 0) */
    float grad_scale;      /* 1 / views accumulated, src/engine/EngineTrainStep.cpp:419-427 */
    int32_t step;          /* bias-correction exponent t >= 1 (the reference passes step + 1) */
    int32_t zero_grad;     /* also clear the gradients, as zero_grad_in_optim does */
} SsbAdamConfig;

/* Replaces fused_optim_3dgs_geometry (src/kernels/optim/FusedGeometryOptim.cu:384-470,
 * kernel :83-380; regulariser weights zero, fp32 state, scalar step) and the two
 * fused_adam_step launches for features_dc and features_sh
 * (src/kernels/optim/FusedAppearanceOptim.cu:59-92) over the splat range
 * [first, first + count).  `m1`/`m2` are the first/second moments.
 * If params->features_sh is NULL the SH part is skipped (see ssb_adam_step_sh_quantized). */
int ssb_adam_step(const SsbSplats* params, const SsbSplats* grads, const SsbSplats* m1, const SsbSplats* m2,
                  int64_t first, int64_t count, const SsbAdamConfig* cfg, void* stream);

/* The optional parts of the reference's optimiser launch that SsbAdamConfig leaves out
 * (src/engine/EngineConfig.h OptimConfig; src/kernels/optim/FusedGeometryOptim.cu:384-470).
 * The regulariser weights are the caller's undivided weights: like the reference's launcher
 * (:457-462) the library divides them by n_total. */
typedef struct SsbAdamExtras {
    float max_gauss_ratio;               /* threshold of the scale-ratio regulariser */
    float scale_regularization_weight;   /* w * (max(max(e^s)/min(e^s), ratio) - ratio) */
    float mcmc_opacity_reg_weight;       /* w * sigmoid(opacity) */
    float mcmc_scale_reg_weight;         /* w * 1e-2 * mean(log-scales) */
    float erank_reg_weight;              /* w * max(-log(erank - 0.99999), 0) */
    float erank_reg_weight_s3;           /* w * smallest normalised squared scale */
    float quat_norm_reg_weight;          /* w * (|q| - 1 - log|q|), evaluated on the normalised quaternion */
    int32_t use_scale_agnostic_mean;     /* FusedGeometryOptim.cu:302-314; needs d_radii */
    const float* d_radii;                /* [n_total] screen radii of ssb_project_fwd (max over the views) */
    const int32_t* d_steps;              /* [n_total] per-splat bias-correction exponents (>= 1), or NULL: cfg->step */
    int64_t n_total;                     /* number of splats of the whole model (the range may be a shard) */
    float* d_densify_score;              /* [n_total] or NULL: |grad_scale * dL/dmean| * exp(largest log-scale) before the
                                            update, the world-gradient densification score (FusedGeometryOptim.cu:283-286) */
} SsbAdamExtras;

/* ssb_adam_step with the optional parts: per-splat regulariser gradients (Slang per_splat_losses_bwd,
 * src/shaders/per_splat_losses.slang:5-141, all five loss cotangents 1), the scale-agnostic mean update and
 * per-splat step counters for every parameter group (steps[idx / stride] in the appearance kernels,
 * src/kernels/optim/FusedAppearanceOptim.cu:34).  extras == NULL is ssb_adam_step. */
int ssb_adam_step_ex(const SsbSplats* params, const SsbSplats* grads, const SsbSplats* m1, const SsbSplats* m2,
                     int64_t first, int64_t count, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream);

/* The same update of means, rotations, scales, opacities and DC with their Adam moments kept in 16-bit joint codes:
 * the non_sh_quant path of fused_optim_3dgs_geometry (src/kernels/optim/FusedGeometryOptim.cu:144-380) on
 * QuantizedAdamState<16, 256> (src/core/Tensor.h:978-1136; pool slots eng.<array>_qfpbo.q / .qb,
 * src/core/PoolSlots.h:107-111).  Per array: d_packed = 4 bytes per cell ((u, log-s) as two uint16), cells = width * splats;
 * d_bounds = one float4 (u min, u max, log-s min, log-s max) per 256 splats.  All-zero buffers are the zero state.  56 bytes of
 * optimiser state per splat instead of 112.  `first` must be a multiple of 256.  As in the reference, the DC regulariser of
 * this path is cfg->sh_reg_weight undivided. */
typedef struct SsbMomentsQ16 {
    uint8_t* d_packed[5];    /* means, quats, scales, opacities, features_dc */
    float* d_bounds[5];
} SsbMomentsQ16;
int ssb_adam_step_q16(const SsbSplats* params, const SsbSplats* grads, const SsbMomentsQ16* moments, int64_t first, int64_t count,
                      const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream);

/* The SH update on the layouts of the reference's fused backward + optimiser at quantisation level 1 (the SH part of
 * fused_projection_bwd_optimizer_3dgs_kernel<..., 256, 8, 16>, src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:709-975; pool
 * slots eng.world.sh_vq16_fpbo and eng.sh_quant_fpbo, src/core/PoolSlots.h:115-120): 8-bit joint state codes (two bytes per cell) and 8- or 16-bit
 * values, with ONE float4 of state bounds and ONE float2 of value bounds per 256 SPLATS, covering all 45 cells of each.  Splats
 * [first_splat, first_splat + n_splats), first_splat a multiple of 256; d_grad is indexed by the global cell (45 * splat + cell).
 * active_sh_degree_plus1 = 0 or 4: all 45 cells are live.  1..3 (the SH degree warm-up): the cells of the bands above the active
 * degree are not updated but written as zero value and zero moments against bounds widened to contain zero, as the reference
 * does (:836-857, :918-925); 1 (degree 0) leaves the buffers untouched.  cfg->sh_reg_weight, grad_scale, zero_grad, step as in
 * ssb_adam_step_sh_quantized; d_steps [n_total] per-splat exponents or NULL. */
int ssb_adam_step_sh_splat_blocks(float* d_grad, uint8_t* d_optim_packed, float* d_optim_bounds, void* d_value_packed, float* d_value_bounds,
                                  int32_t value_bits, int64_t first_splat, int64_t n_splats, int64_t n_total, int32_t active_sh_degree_plus1,
                                  const SsbAdamConfig* cfg, const int32_t* d_steps, void* stream);

/* Replaces fused_adam_step (src/kernels/optim/FusedAppearanceOptim.cu:11-92) on one array of numel floats, `stride` per
 * splat: Adam with the decoupled-offset L2 term 2 * l2_reg / numel * (max(x - off, 0) + min(x + off, 0)), bias correction from
 * `step`, or per splat from d_steps [numel / stride] when given.  ssb_adam_step covers the six arrays of a splat set in one
 * call (and leaves out features_dc when params->features_dc is NULL); this entry is the reference's granularity. */
int ssb_adam_plain(float* d_param, float* d_grad, float* d_m1, float* d_m2, int64_t numel, int32_t stride, float lr, int32_t step,
                   const int32_t* d_steps, float l2_reg, float l2_reg_offset, float grad_scale, int32_t zero_grad, void* stream);

/* Replaces fused_adam_step_quantized_value (src/kernels/optim/FusedAppearanceOptim.cu:421-479,
 * kernel :291-418): Adam on SH coefficients whose values live in a QuantizedTensor
 * <value_bits,256> and whose state lives in a QuantizedAdamState<8,256>
 * (src/core/Tensor.h:978-1136).  `numel` cells starting at cell `first_cell`,
 * which must be a multiple of 256.  d_grad is fp32 [cells].
 * value_bits = 32 replaces fused_adam_step_quantized (FusedAppearanceOptim.cu:137-271) instead: the
 * values are plain fp32 (d_value_packed is a float array, d_value_bounds may be NULL) and only the
 * state is quantised. */
int ssb_adam_step_sh_quantized(float* d_grad, uint8_t* d_optim_packed, float* d_optim_bounds,
                               void* d_value_packed, float* d_value_bounds, int32_t value_bits,
                               int64_t first_cell, int64_t numel, int64_t numel_total,
                               const SsbAdamConfig* cfg, void* stream);

/* The same with the two remaining options of the reference's launchers (FusedAppearanceOptim.cu:232-271,421-479):
 * optim_bits = 4 stores the state as QuantizedAdamState<4,256> (one byte per cell, u in the low nibble;
 * src/core/Tensor.h:1051-1054,1091-1095) instead of 8 (two bytes per cell); d_steps != NULL gives per-splat
 * step counters, cell c using d_steps[c / cells_per_splat] (steps[idx / stride], :166,330).
 * optim_bits = 8 and d_steps == NULL is the call above. */
int ssb_adam_step_sh_quantized_ex(float* d_grad, uint8_t* d_optim_packed, float* d_optim_bounds,
                                  void* d_value_packed, float* d_value_bounds, int32_t value_bits, int32_t optim_bits,
                                  int64_t first_cell, int64_t numel, int64_t numel_total,
                                  const SsbAdamConfig* cfg, const int32_t* d_steps, int32_t cells_per_splat, void* stream);

/* QuantizedTensor<BITS,256>::encode_v / decode_v over whole buffers
 * (src/core/Tensor.h:1366-1393); bounds = float2 per 256 cells. */
int ssb_quant_encode(const float* d_values, int64_t numel, int32_t bits, void* d_packed, float* d_bounds, void* stream);
int ssb_quant_decode(const void* d_packed, const float* d_bounds, int64_t numel, int32_t bits, float* d_values, void* stream);

/* ---- one training iteration --------------------------------------------- */

/* ---------------------------------------------------------------------------
 * Gradient reduction and parameter distribution between the GPUs of one node, over peer memory.
 * Reference: the sum of the sub-batches' gradients and the single optimiser pass of
 * _engine_train_step_split_one_per_camera (src/engine/EngineTrainStep.cpp:366-427), which the reference
 * does on one GPU.  Here the views of a batch are split between ranks (one process per GPU), each
 * rank owns a contiguous range of splats, and per iteration it
 *   1. ssb_peer_reduce_f32: adds the peers' partial gradients of its range to its own (plain loads
 *      from their memory over NVLink);
 *   2. runs ssb_adam_step / ssb_adam_step_sh_quantized on the range;
 *   3. ssb_peer_broadcast: stores the range's updated parameters into every peer's replica.
 * The caller must order the ranks with a barrier before 1 (all backward passes complete) and after 3
 * (all replicas complete); no kernel waits on another GPU.
 *
 * A table names up to SSB_MAX_PEER_BUFFERS buffers that have the same layout on every rank
 * (base[b][r] = rank r's copy of buffer b as mapped in THIS process) and up to
 * SSB_MAX_PEER_SEGMENTS byte ranges of them; a segment must start on a 16-byte boundary.
 * Buffers come from ssb_peer_alloc (a zeroed device allocation that can be exported), are exported
 * with ssb_peer_export (a 64-byte CUDA IPC handle to send to the other processes) and mapped there
 * with ssb_peer_open / unmapped with ssb_peer_close. */
enum { SSB_MAX_PEERS = 8, SSB_MAX_PEER_BUFFERS = 4, SSB_MAX_PEER_SEGMENTS = 12, SSB_PEER_HANDLE_BYTES = 64 };
typedef struct SsbPeerSegment {
    int32_t buffer;
    int32_t pad;
    int64_t offset_bytes;
    int64_t bytes;
} SsbPeerSegment;
typedef struct SsbPeerTable {
    int32_t world, self, n_segments, pad;
    void* base[SSB_MAX_PEER_BUFFERS][SSB_MAX_PEERS];
    SsbPeerSegment seg[SSB_MAX_PEER_SEGMENTS];
    /* Optional: the NVSwitch multicast address of each buffer (one address that reaches every rank's
     * copy).  When it is non-NULL for every buffer a table uses, the sum is taken inside the switch
     * (multimem.ld_reduce: each rank receives its range once instead of once per peer) and the
     * broadcast is one multicast store (multimem.st).  NULL: plain loads and stores per peer. */
    void* multicast[SSB_MAX_PEER_BUFFERS];
} SsbPeerTable;
int ssb_peer_alloc(int64_t bytes, void** d_ptr);
int ssb_peer_free(void* d_ptr);
int ssb_peer_export(const void* d_ptr, unsigned char handle[SSB_PEER_HANDLE_BYTES]);
int ssb_peer_open(const unsigned char handle[SSB_PEER_HANDLE_BYTES], void** d_ptr);
int ssb_peer_close(void* d_ptr);
/* own[segment] += sum over the other ranks of theirs[segment]; fp32 data. */
int ssb_peer_reduce_f32(const SsbPeerTable* table, void* stream);
/* theirs[segment] = own[segment] for every other rank; any data. */
int ssb_peer_broadcast(const SsbPeerTable* table, void* stream);

/* The three steps above as ONE pass: reduce-scatter, Adam and all-gather fused.  For its range of splats
 * [first, first + count) the calling rank reads every other rank's partial gradients straight into the optimiser
 * kernels (summed in registers, never written back), updates parameters and moments, and stores every updated
 * parameter into all replicas, so inbound gradient traffic and outbound parameter traffic share the NVLink time and the
 * range's gradients make one trip instead of three.  Plain peer loads and stores only.
 *
 * replicas: every rank's copy of the exchanged allocations as mapped in this process ([self] = this rank's own):
 * `grads` holds all six gradient arrays of `grads`, `params` all parameter arrays of `params` (with the same layout on
 * every rank), `sh_packed` / `sh_bounds` the quantised SH codes and their bounds (NULL when SH is fp32 inside params).
 * Optimiser state (m1, m2, sh_state->d_optim_*) is local to the owning rank.  With quantised SH a rank's range must
 * cover whole 256-cell blocks (ranges in multiples of 256 splats).  world == 1 is the plain optimiser step.
 * The caller orders the ranks before (all backward passes complete) and after (all replicas complete) the call;
 * ssb_exchange_step does both.  Reference: the gradient sum over sub-batches and the single optimiser pass of
 * _engine_train_step_split_one_per_camera (src/engine/EngineTrainStep.cpp:366-427), done there on one GPU. */
typedef struct SsbPeerReplicas {
    int32_t world, self;
    void* grads[SSB_MAX_PEERS];
    void* params[SSB_MAX_PEERS];
    void* sh_packed[SSB_MAX_PEERS];
    void* sh_bounds[SSB_MAX_PEERS];
    /* Optional NVSwitch multicast address of each allocation (one address that reaches every rank's copy; NULL = none).
     * When every exchanged allocation has one, gradients are read with multimem.ld_reduce (the switch adds the ranks'
     * copies: a rank receives its range once instead of once per peer) and parameters are written with multimem.st (one
     * store lands in every replica).  Per NVLink direction a GPU then moves about two thirds of the bytes. */
    void* mc_grads;
    void* mc_params;
    void* mc_sh_packed;
    void* mc_sh_bounds;
} SsbPeerReplicas;
/* Quantised SH values and optimiser state of ssb_adam_step_sh_quantized_ex, as one argument. */
typedef struct SsbShAdamState {
    uint8_t* d_optim_packed;
    float* d_optim_bounds;
    void* d_value_packed;
    float* d_value_bounds;
    int32_t value_bits;    /* 8, 16, or 32 (fp32 values, quantised state) */
    int32_t optim_bits;    /* 8 (0 means 8) or 4 */
    int32_t layout;        /* SSB_SH_LAYOUT_CELL_BLOCKS (0): one bound per 256 cells, the layout of fused_adam_step_quantized_value;
                            * SSB_SH_LAYOUT_SPLAT_BLOCKS: one bound per 256 splats (ssb_adam_step_sh_splat_blocks), taken by
                            * ssb_project_bwd_optimize and ssb_step_backward_optimize only */
} SsbShAdamState;
enum { SSB_SH_LAYOUT_CELL_BLOCKS = 0, SSB_SH_LAYOUT_SPLAT_BLOCKS = 1 };
int ssb_reduce_adam_broadcast(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                              const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                              int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg,
                              const SsbAdamExtras* extras, void* stream);

/* The same with the moments of means, rotations, scales, opacities and DC in 16-bit codes (SsbMomentsQ16, see
 * ssb_adam_step_q16): m1 / m2 then only carry features_sh and may be NULL when sh_state is given.  A rank's range must start
 * on a multiple of 256 splats (the codes' bounds are per block of 256); gradients and parameters move by per-peer loads and
 * stores (the multicast kernels keep fp32 moments). */
int ssb_reduce_adam_broadcast_q16(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                                  const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                                  int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg,
                                  const SsbAdamExtras* extras, void* stream);

/* barrier, ssb_reduce_adam_broadcast, barrier.  `barrier(ctx, stream)` must return 0 once every rank has reached it,
 * ordered on `stream` (an NCCL all-reduce of one element enqueued on the stream does that), and non-zero when a rank
 * is missing or the wait timed out: ssb_exchange_step then returns SSB_ERR_PEER -- before the exchange nothing has been
 * launched, so no kernel ever waits for a rank that is not coming. */
typedef int (*SsbBarrierFn)(void* ctx, void* stream);
int ssb_exchange_step(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                      const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                      int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras,
                      SsbBarrierFn barrier, void* barrier_ctx, void* stream);
int ssb_exchange_step_q16(const SsbPeerReplicas* replicas, const SsbSplats* params, const SsbSplats* grads,
                          const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                          int64_t first, int64_t count, int64_t n_total, const SsbAdamConfig* cfg, const SsbAdamExtras* extras,
                          SsbBarrierFn barrier, void* barrier_ctx, void* stream);

/* Owns every intermediate buffer of an iteration (the reference keeps them in
 * its process-global DevicePool, src/core/Tensor.h:151-351) and runs, per view,
 * projection -> keys -> sort -> ranges -> raster -> loss -> raster bwd ->
 * projection bwd, accumulating gradients exactly like the reference's
 * one-camera-per-sub-batch loop (src/engine/EngineTrainStep.cpp:287-437). */
typedef struct SsbStep SsbStep;

typedef struct SsbStepConfig {
    int64_t n_splats;
    int32_t width, height;
    int32_t camera_model;
    int32_t antialiased;
    int64_t isect_capacity;  /* max (splat, tile) pairs per view; 0 = 12 * n_splats */
    float w_l1, w_ssim;      /* 0.8 / 0.2 in the benchmark configuration */
} SsbStepConfig;

int ssb_step_create(const SsbStepConfig* cfg, SsbStep** out);
void ssb_step_destroy(SsbStep* step);
int64_t ssb_step_device_bytes(const SsbStep* step);

/* ---- splat.ply: the inference artefact written next to a checkpoint -------------------------------------------------
 * ssb_ply_write restates the PLY part of engine_save_checkpoint (src/engine/EngineCheckpoint.cpp:130-330): the property
 * layout of the original 3D Gaussian Splatting release (x y z, nx ny nz = 0, f_dc_0..2, f_rest_0..44 channel-major, opacity,
 * scale_0..2, rot_0..3; binary little endian floats, raw values), without the splats that have a non-finite parameter or an
 * opacity logit below -5.5373, SH values dequantised when shq names 8- or 16-bit codes.  The kept splats keep their order.
 * Rows are assembled on the device and streamed through pinned staging; the call synchronises `stream`.
 * *kept (may be NULL) receives the number of vertices written.
 * ssb_ply_info / ssb_ply_read restate read_splat_ply (src/checkpoint/SplatPly.cpp:159-254): vertex properties in any order
 * and scalar type, binary little endian or ASCII; SSB_ERR_UNSUPPORTED for a file that is not a splat PLY.  The caller
 * sizes HOST arrays from ssb_ply_info (features_sh: [num][(sh_degree + 1)^2 - 1][3], coefficient-major, or NULL to skip
 * the f_rest columns). */
int ssb_ply_write(const char* path, const SsbSplats* params, const SsbShQuant* shq, int64_t n, int64_t* kept, void* stream);
int ssb_ply_info(const char* path, int64_t* num, int32_t* sh_degree);
int ssb_ply_read(const char* path, int64_t num, int32_t sh_degree, float* h_means, float* h_quats, float* h_scales, float* h_opacities,
                 float* h_features_dc, float* h_features_sh);

/* Makes every view's projection fold the splats' view radii (view_radius_3dgs, src/shaders/projection_utils.slang:1033-1043)
 * into d_radii [n_splats] by maximum, as ssb_project_fwd does with its d_radii argument: the array the scale-agnostic mean
 * update, the scale clip, the score update and the revised noise read.  The caller zeroes it once per iteration.  NULL: off. */
int ssb_step_set_radii(SsbStep* step, float* d_radii);

/* The SH degree the step's projections evaluate (0..3; default 3): the reference's trainer raises it by one every
 * sh_degree_warmup_every iterations (sh_degree_to_use = step / sh_degree_warmup_every, src/app/TrainerCore.cpp:948) and calls
 * the Vanilla3DGS<degree> instantiation; bands above it are neither read nor given a gradient, so their Adam state stays put. */
int ssb_step_set_sh_degree(SsbStep* step, int32_t sh_degree);

/* The lens-distortion tier of the step's cameras (SsbCameras::distortion; the engine's camera.distortion with
 * dist_coeffs[C][8], src/engine/EngineTrainStep.cpp) and its coefficient rows: row v belongs to view v of the NEXT
 * ssb_step_views / ssb_step_views_gated call (the same indexing as that call's d_viewmats), and for
 * ssb_step_backward_optimize to view v of the views it is given.  The pointer is read at enqueue time and the rows on the
 * device when the views run.  tier SSB_DISTORTION_NONE (the default) ignores d_dist_coeffs.  A (model, tier) pair the
 * projection does not build is SSB_ERR_UNSUPPORTED here. */
int ssb_step_set_distortion(SsbStep* step, int32_t tier, const float* d_dist_coeffs);

/* Switches the densification outputs of the step on (accum_mode != SSB_ACCUM_NONE) or off: every view then also
 * builds its SSIM loss map (ssim_loss_map_weight * (1 - SSIM variant), as ssb_loss_l1_ssim_fwdbwd_map on a zeroed map;
 * the reference adds its per-pixel loss map of the pixel-loss pass on top, src/engine/EngineLoss.cpp, which is not
 * built here) and the raster backward pass folds it into d_accum_weight [n_splats] (and d_accum_weight_den for
 * SSB_ACCUM_AVG) as ssb_raster_bwd_accum does.  The arrays are combined into across views and calls
 * (EngineTrainStep.cpp:264-272); the caller zeroes them.  Allocates one [H][W] map per lane on first use. */
int ssb_step_set_densify(SsbStep* step, int32_t ssim_loss_map_mode, float ssim_loss_map_weight, int32_t accum_mode,
                         float* d_accum_weight, float* d_accum_weight_den);

/* Makes every view of the step use the general loss (ssb_loss_multi_scale) with cfg's num_scales, loss_map_mode and
 * mask; w_l1 / w_ssim stay the step's.  cfg->d_mask, if given, holds one mask per view of the following ssb_step_views
 * calls, [n_views][mask_h][mask_w], indexed like d_gt.  With densification outputs switched on (ssb_step_set_densify)
 * and loss_map_mode != 0 the per-splat weights are gathered from this loss map (the reference's path:
 * src/engine/EngineLoss.cpp:852-862) instead of the SSIM-only map.  cfg == NULL switches back to the one-scale,
 * unmasked loss.  With a mask the step also builds each view's live-tile map (ssb_tile_active) and leaves the tiles that
 * no term of the loss reads out of the intersection, as the reference does when it has a mask and no alpha supervision
 * (src/engine/EngineTrainStep.cpp:84-126).  Allocates the pyramid workspace per lane. */
int ssb_step_set_loss(SsbStep* step, const SsbLossConfig* cfg);

/* Forward + loss + backward of `n_views` views (device camera arrays and device
 * targets d_gt [n_views][H][W][3]); gradients are overwritten by the first view
 * when `accumulate` == 0 and added to otherwise.  Loss sums accumulate into
 * d_losses[3] (device; caller zeroes). */
int ssb_step_views(SsbStep* step, const SsbSplats* params, const SsbShQuant* shq,
                   const float* d_viewmats, const float* d_intrins, const float* d_gt, int32_t n_views,
                   const SsbSplats* grads, int accumulate, float* d_losses, void* stream);
/* The same, for targets that are still arriving: gt_ready[v] (a cudaEvent_t, or NULL) is waited for on
 * the device just before view v's loss kernel, the first stage that reads its target image.  Projection,
 * intersection and rasterisation of a view therefore overlap the host-to-device copy of its target, and
 * one call covers a whole batch whose targets are copied view by view on another stream.
 * gt_ready may be NULL (no gating).  No counterpart in the reference, whose targets are resident. */
int ssb_step_views_gated(SsbStep* step, const SsbSplats* params, const SsbShQuant* shq,
                         const float* d_viewmats, const float* d_intrins, const float* d_gt, int32_t n_views,
                         void* const* gt_ready, const SsbSplats* grads, int accumulate, float* d_losses, void* stream);

/* Projection backward of ALL views fused with the optimiser, on caller buffers (the reference's
 * fused_projection_bwd_optimizer_3dgs in its unpacked mode, src/kernels/optim/FusedProjectionBwdOptim.cu:76-213, kernel
 * FusedProjectionBwdOptim_kernel.cuh:146-1030): d_aabb [views][n][4] and d_v_screen [views][n] as the forward passes and the
 * rasteriser's backward passes left them, cams->count views.  Splats are worked through in ranges of 131072: the projection
 * backward of every view writes the range's gradients into the workspace (ssb_project_bwd_optimize_workspace_bytes(n), 256-byte
 * aligned; it stays in L2), the Adam kernels (ssb_adam_step_ex, and ssb_adam_step_sh_quantized_ex when sh_state is given)
 * read them from there, so no world-gradient array exists.  The result equals ssb_project_bwd over all views followed by the
 * unfused optimiser calls.  cfg->grad_scale scales the gradients as there; cfg->zero_grad is ignored. */
int64_t ssb_project_bwd_optimize_workspace_bytes(int64_t n);
int ssb_project_bwd_optimize(const SsbSplats* params, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                             const SsbScreenRec* d_v_screen, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                             const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* d_workspace, int64_t workspace_bytes, void* stream);
/* The same with the moments of means, rotations, scales, opacities and DC in 16-bit codes (SsbMomentsQ16, see ssb_adam_step_q16):
 * the reference's stock configuration of this kernel (quantisation level 1 with NonShQuantState::enabled).  m1 / m2 then only
 * carry features_sh and may be NULL when sh_state is given.  The DC regulariser is the fused kernel's, 2 w / (3 n) with the dead
 * zone (FusedProjectionBwdOptim_kernel.cuh:355-358, :1137), not the undivided w of the unfused kernel. */
int ssb_project_bwd_optimize_q16(const SsbSplats* params, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                                 const SsbScreenRec* d_v_screen, const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2,
                                 const SsbShAdamState* sh_state, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* d_workspace,
                                 int64_t workspace_bytes, void* stream);

/* Projection backward of all views fused with the optimiser: the reference's use_fused_proj_bwd_optim path
 * (fused_projection_bwd_optimizer_3dgs_kernel, src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:146-1030: one
 * thread per splat loops over its views, so the world gradients are never stored).
 *   ssb_step_set_fused_backward(step, max_views > 0): ssb_step_views[_gated] then stops after each view's raster backward
 *     and keeps the view's aabb and screen-gradient records ((16 + 48) bytes per splat and view); `grads`, `accumulate`
 *     are ignored.  Views of successive calls are appended until ssb_step_backward_optimize consumes them.  0 switches back.
 *   ssb_step_backward_optimize: for one range of 131 072 splats after the other, the projection backward over all kept
 *     views (a thread per splat, gradients summed in registers and shared memory) writes the range's gradients to a
 *     31 MB scratch that the Adam kernels of the same range read straight back out of L2.  d_viewmats / d_intrins are the
 *     cameras of the kept views in the order they were given; n_views must equal their number.  m1 / m2 / cfg / extras
 *     as for ssb_adam_step_ex (cfg->zero_grad is ignored); sh_state != NULL runs the quantised SH update of
 *     ssb_adam_step_sh_quantized_ex on it (then params->features_sh, m1/m2->features_sh may be NULL), else SH is
 *     part of the plain update.  With sh_state->layout = SSB_SH_LAYOUT_CELL_BLOCKS the state layouts are those of the unfused
 *     optimiser calls, so the two paths can be mixed from one iteration to the next; SSB_SH_LAYOUT_SPLAT_BLOCKS is the
 *     layout the reference keeps for its fused path (ssb_adam_step_sh_splat_blocks; shq->bounds_stride is then 0).
 *   ssb_step_backward_optimize_q16: the same with the moments of the five non-SH arrays in 16-bit codes
 *     (ssb_project_bwd_optimize_q16).
 * The result equals ssb_step_views + ssb_adam_step_* up to the order of the floating-point sums over views. */
int ssb_step_set_fused_backward(SsbStep* step, int32_t max_views);
int ssb_step_backward_optimize(SsbStep* step, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmats, const float* d_intrins,
                               int32_t n_views, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state, const SsbAdamConfig* cfg,
                               const SsbAdamExtras* extras, void* stream);
int ssb_step_backward_optimize_q16(SsbStep* step, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmats, const float* d_intrins,
                                   int32_t n_views, const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2,
                                   const SsbShAdamState* sh_state, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream);

/* Pair count M of the last view processed (host copy taken after that view's
 * kernels finished; synchronises the stream). */
int ssb_step_last_isects(SsbStep* step, int64_t* h_n_isects, void* stream);

/* The largest per-view pair count since the step was created or this word was last cleared, kept on the
 * device so that an iteration needs no host synchronisation to stay safe: a view with more pairs than
 * isect_capacity renders from clamped lists (ssb_intersect_tiles) and the count shows it.
 * ssb_step_max_pairs_device returns the device address of that int64 (valid for the step's lifetime) so a
 * caller can copy it to the host together with its loss scalars; ssb_step_status copies it to *h_max_pairs
 * (may be NULL), clears it when `reset` != 0, synchronises the stream and returns SSB_ERR_CAPACITY when a
 * view exceeded the capacity.  The reference needs neither: it reads M back every view and sizes its
 * buffers exactly (src/kernels/tile/IntersectTile.cu:432-459). */
const int64_t* ssb_step_max_pairs_device(const SsbStep* step);
int64_t ssb_step_isect_capacity(const SsbStep* step);
int ssb_step_status(SsbStep* step, int64_t* h_max_pairs, int reset, void* stream);

/* One image, forward only: projection, tile intersection and the forward rasteriser for one camera of the step's size and
 * model (with the step's SH degree and distortion tier; row 0 of the distortion rows), into caller buffers -- what the
 * reference's viewer asks of forward_3dgs + engine_copy_render_to_host (src/app/webviewer/RenderWorker.cpp:285-300).
 * d_rgb [H][W][3]; d_depth [H][W] ray depth normalised by 1 - T, or NULL; d_T [H][W] transmittance, or NULL.  Uses the
 * buffers of the step's first lane, ordered after views already enqueued and before views enqueued later; nothing is
 * allocated.  The display transforms of the viewer (alpha, depth scaling, normals, 8-bit) stay with the caller. */
int ssb_step_render(SsbStep* step, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmat, const float* d_intrin,
                    float* d_rgb, float* d_depth, float* d_T, void* stream);

/* Device buffers of the last view, for inspection by tests: any pointer may be
 * NULL.  Valid until the next ssb_step_views / ssb_step_destroy. */
int ssb_step_peek(SsbStep* step, const float** d_rgb, const float** d_depth, const float** d_T,
                  const int32_t** d_last_ids, const SsbScreenRec** d_screen, const float** d_aabb);

/* Per-stage device timing of ssb_step_views (CUDA events on the stream the
 * kernels run on).  Off by default.  ssb_step_get_profile synchronises, adds
 * the views recorded since the last call into ms[SSB_STAGE_COUNT] (milliseconds
 * summed over views), stores how many views that was, and resets. */
enum { SSB_STAGE_PROJECT_FWD = 0, SSB_STAGE_TILE_KEYS, SSB_STAGE_SORT, SSB_STAGE_TILE_RANGES, SSB_STAGE_RASTER_FWD,
       SSB_STAGE_LOSS, SSB_STAGE_RASTER_BWD, SSB_STAGE_PROJECT_BWD, SSB_STAGE_COUNT };
int ssb_step_set_profiling(SsbStep* step, int enable);
int ssb_step_get_profile(SsbStep* step, float* ms, int32_t* n_views);

/* ------------------------------------------------------------------------- *
 * Checkpoint container (state.tar)
 *
 * Replaces engine_save_checkpoint / engine_load_checkpoint's file handling
 * (src/engine/EngineCheckpoint.cpp:350-474) and the helpers of src/core/CheckpointIO.h:
 * a POSIX ustar archive whose first member is "state.json" and whose other members are
 * "<buffer name>.npy", each a flat one-dimensional NPY v1.0 array.  Files written here are
 * byte-for-byte what the reference writes for the same names, sizes and contents, and the
 * reader takes the reference's files.  Which buffers go in, and under which names, is the
 * caller's business (the reference's names are listed in src/core/PoolSlots.h:88-125).
 *
 * `dtype` is one of SsbDType, numbered like the reference's NpyScalar tags
 * (src/core/Tensor.h:26).  nbytes must be a multiple of the element size.  Names are at
 * most 99 bytes.  Device arrays are staged through two pinned 32 MiB buffers so the
 * copy and the file access overlap; no device memory is allocated.  The functions
 * synchronise `stream` before they return.
 * ssb_ckpt_read_device / ssb_ckpt_read_host return SSB_ERR_CAPACITY when the stored array
 * does not have exactly nbytes bytes (the reference throws "size mismatch"), and
 * SSB_ERR_INVALID_ARGUMENT when there is no member of that name.
 * ssb_ckpt_read_bytes with buf == NULL only reports the member's size.
 * ------------------------------------------------------------------------- */
typedef enum SsbDType { SSB_DTYPE_U1 = 0, SSB_DTYPE_U2, SSB_DTYPE_U4, SSB_DTYPE_U8, SSB_DTYPE_I4, SSB_DTYPE_I8,
                        SSB_DTYPE_F2, SSB_DTYPE_F4, SSB_DTYPE_F8, SSB_DTYPE_B1 } SsbDType;
/* The two headers on their own, for a caller that streams its own archive: the NPY header of a flat array
 * (returns its length in bytes, a multiple of 64, or a negative status) and the 512-byte member header. */
int ssb_ckpt_array_header(int dtype, uint64_t numel, void* out, int capacity);
int ssb_ckpt_member_header(const char* name, uint64_t size, void* out512);
typedef struct SsbCkptWriter SsbCkptWriter;
typedef struct SsbCkptReader SsbCkptReader;
int ssb_ckpt_writer_open(const char* path, SsbCkptWriter** out);
int ssb_ckpt_write_bytes(SsbCkptWriter* w, const char* name, const void* data, uint64_t size);
int ssb_ckpt_write_host(SsbCkptWriter* w, const char* name, const void* h_ptr, uint64_t nbytes, int dtype);
int ssb_ckpt_write_device(SsbCkptWriter* w, const char* name, const void* d_ptr, uint64_t nbytes, int dtype, void* stream);
int ssb_ckpt_writer_close(SsbCkptWriter* w);   /* writes the end-of-archive blocks, closes the file and frees w */
int ssb_ckpt_reader_open(const char* path, SsbCkptReader** out);
int ssb_ckpt_member_count(const SsbCkptReader* r);
int ssb_ckpt_member_info(const SsbCkptReader* r, int index, char* name, int name_capacity, uint64_t* size);
int ssb_ckpt_read_bytes(SsbCkptReader* r, const char* name, void* buf, uint64_t capacity, uint64_t* size);
int ssb_ckpt_array_info(SsbCkptReader* r, const char* name, char* descr, int descr_capacity, uint64_t* data_bytes);
int ssb_ckpt_read_host(SsbCkptReader* r, const char* name, void* h_ptr, uint64_t nbytes);
int ssb_ckpt_read_device(SsbCkptReader* r, const char* name, void* d_ptr, uint64_t nbytes, void* stream);
int ssb_ckpt_reader_close(SsbCkptReader* r);

/* ------------------------------------------------------------------------- *
 * Densification: the part that runs on every training step
 *
 * Replaces, for the 3dgs primitive, what engine_densify_step does outside its periodic relocation
 * (src/engine/EngineDensify.cpp:193-263,355-367):
 *   ssb_densify_update_scores = densify_clip_scale_tensor + densify_accum_finalize_tensor + densify_update_weight +
 *     densify_clip_score_tensor (src/kernels/densify/DensifyScoring.cu:150-409, quantile: src/kernels/densify/Quantile.cu).
 *     d_radii [n] the largest screen radius of the step (as the optimiser's extras take it); d_scales [n][3] log-scales,
 *     clipped in place; d_accum_weight [n] (and d_accum_weight_den [n] for SSB_ACCUM_AVG) the per-splat weights the raster
 *     backward pass gathered (ssb_raster_bwd_accum), turned into their quotient in place for SSB_ACCUM_AVG;
 *     d_world_grad_score [n] or NULL the score the optimiser wrote (SsbAdamExtras::d_densify_score), blended in
 *     geometrically with weight score_blend_world_grad (1: it alone); with neither, the score is sigmoid(opacity) times
 *     d_opacities; d_accum_buffer [n][2] the running (score, steps) pair, NULL to only clip the scales;
 *     d_sample_score [n][2] or NULL gets (clipped score ^ final_score_power, steps).
 *     score_mode: 0 mean, 1 max, 2 median (a hash-driven random walk), 3 geometric mean (DensifyScoreMode,
 *     src/kernels/densify/Densify.cuh:10-15).  score_clip_quantile in (0, 1) clips the accumulator at that quantile of
 *     its strictly positive finite entries, copies of the maximum left out; it needs the workspace.
 *     INFINITY switches max_screen_size / max_screen_size_clip_hardness / max_world_size off.
 *   ssb_densify_add_noise = mcmc_add_noise_tensor (revised == 0) or revised_add_noise_tensor
 *     (src/kernels/densify/McmcRelocation.cu:556-654, src/shaders/densify.slang:13-74).  The three normals come from a hash
 *     of the splat's own parameters, so the result is a function of the input; the hash amplifies rounding differences, so
 *     it equals the reference's in distribution, not number for number.
 * ------------------------------------------------------------------------- */
typedef struct SsbDensifyScoreConfig {
    float max_screen_size, max_screen_size_clip_hardness, max_world_size;
    int32_t accum_mode;              /* SSB_ACCUM_* the raster weights were gathered with */
    int32_t score_mode;
    float score_blend_world_grad, score_power, score_clip_quantile, final_score_power;
} SsbDensifyScoreConfig;
int64_t ssb_densify_workspace_bytes(int64_t n_splats);
int ssb_densify_update_scores(const SsbDensifyScoreConfig* cfg, int64_t n_splats, const float* d_radii, float* d_scales, const float* d_opacities,
                              float* d_accum_weight, const float* d_accum_weight_den, const float* d_world_grad_score, float* d_accum_buffer,
                              float* d_sample_score, void* d_workspace, int64_t workspace_bytes, void* stream);
int ssb_densify_add_noise(int64_t n_splats, float scaler, int32_t revised, const float* d_radii, float* d_means, const float* d_scales,
                          const float* d_quats, const float* d_opacities, void* stream);

/* The periodic part of the revised strategy: relocate_splats_with_long_axis_split_tensor and
 * add_splats_with_long_axis_split_tensor (src/kernels/densify/Relocation.cu:205-369; split rule
 * src/shaders/densify.slang:76-94; draw src/kernels/densify/DensifySampling.cu:278-390).
 *   ssb_densify_relocate: a splat is dead when sigmoid(opacity) <= min_opacity or its parameters are not finite.  As many
 *     live splats as there are dead ones are drawn without replacement with probability proportional to the score
 *     (d_sample_score, else d_accum_buffer: [.][2], the score in lane 0; Efraimidis-Spirakis keys from the integer hash
 *     of (seed, index), the smallest keys win); each drawn splat is split along its longest axis into itself and one
 *     dead slot: means moved apart by half the longest extent, the long axis halved and the others scaled by 0.85,
 *     opacity logit(k / (1 + e^-o - k))-style reduced with k = split_opacity_k, rotation, DC and SH copied (quantised
 *     SH values are decoded with the source block's bounds and encoded against the destination block's current ones),
 *     the destination's optimiser state set to zero (quantised state: the codes nearest to zero), its step counter
 *     cleared, its score copied.  The number of dead splats stays on the device; *d_num_relocated (device, may be NULL)
 *     receives it.  Dead slots are filled in ascending order (the reference's order varies from run to run).
 *   ssb_densify_add: num_new live splats are drawn the same way (no splat is excluded) and split into themselves and
 *     the slots cur_n .. cur_n + num_new - 1, which the arrays must have room for.
 * Arrays: params / m1 / m2 as for the optimiser; an array that is NULL is not kept in that form (SH values NULL when
 * they are quantised in sh.d_value_packed; SH moments NULL when sh.d_optim_packed holds the quantised state).
 * Bounds are one per 256 cells.  The workspace serves both calls and depends on cur_n only. */
typedef struct SsbDensifyState {
    SsbSplats params, m1, m2;
    SsbShAdamState sh;             /* d_optim_packed NULL: fp32 SH moments; d_value_packed NULL or value_bits 32: fp32 SH values */
    float* d_accum_buffer;         /* [capacity][2] running (score, steps), or NULL */
    const float* d_sample_score;   /* [capacity][2] or NULL: then d_accum_buffer drives the draw */
    int32_t* d_steps;              /* per-splat step counters, or NULL */
} SsbDensifyState;
int64_t ssb_densify_relocate_workspace_bytes(int64_t n_splats);
int ssb_densify_relocate(const SsbDensifyState* state, int64_t cur_n, float min_opacity, float split_opacity_k, uint32_t seed, void* d_workspace,
                         int64_t workspace_bytes, int32_t* d_num_relocated, void* stream);
int ssb_densify_add(const SsbDensifyState* state, int64_t cur_n, int64_t num_new, float split_opacity_k, uint32_t seed, void* d_workspace,
                    int64_t workspace_bytes, void* stream);

/* Number of kernel launches the library has issued from this process so far. */
int64_t ssb_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SSB_H_ */
