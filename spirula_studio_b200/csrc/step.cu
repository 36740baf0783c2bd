// One training iteration's forward + loss + backward over a batch of views.
//
// Host-side orchestration in the shape of the reference's
// one-camera-per-sub-batch loop (src/engine/EngineTrainStep.cpp:287-437, which
// calls forward_3dgs, src/engine/EngineForward.cpp:24-311, then _engine_loss,
// src/engine/EngineLoss.cpp:439-902, per camera and runs the optimiser once).
// The SsbStep object owns the intermediate buffers the reference keeps in its
// DevicePool; they are sized once for (n_splats, width, height, capacity) and
// reused for every view, so a step performs no allocation and no host
// synchronisation: the (splat, tile) pair count stays on the device.
//
// Views are independent until their gradients are added, so the object keeps
// THREE sets of per-view buffers ("lanes") and runs consecutive views round-robin on three
// internal streams: the latency-bound stages of one view (key generation, sort,
// projection backward) fill the issue slots the arithmetic-bound rasteriser of
// the others leave idle.  The projection backward of view v waits for that of
// view v-1, so gradients are accumulated in view order exactly as the serial
// loop does.  The caller's stream is joined on both sides: everything it
// enqueued before the call is visible to the lanes, and everything the lanes do
// is complete before work it enqueues afterwards.
#include "ssb_common.cuh"

#include <new>

enum { SsbStep_kMaxProfViews = 64, SsbStep_kLanes = 3 };

struct SsbLane {
    float* aabb;          // [n][4]
    float* depths;        // [n]
    SsbScreenRec* screen; // [n]
    SsbScreenRec* v_screen;
    void* isect_ws;       // tile cursors + the unsorted (depth, pair) words
    int32_t* flat;        // sorted pair indices
    int64_t* n_isects;    // device
    int32_t* offsets;     // [tiles]
    float* rgb; float* T; int32_t* last_ids; float* v_rgb;
    float* loss_map;      // [P], only with ssb_step_set_densify
    void* loss_ws;        // pyramid of the general loss, only with ssb_step_set_loss
    int32_t* tile_live;   // [tiles] live-tile map of the view's mask, only with a mask in ssb_step_set_loss
    cudaStream_t stream;
    cudaEvent_t bwd_done;  // this lane's last projection backward
    cudaEvent_t all_done;
};

struct SsbStep {
    SsbStepConfig cfg;
    int tw, th;
    int64_t capacity;
    int64_t bytes;
    int64_t isect_ws_bytes;
    int n_lanes;
    int last_lane;
    SsbLane lane[SsbStep_kLanes];
    cudaEvent_t fork;
    // optional per-stage timing (views then run one after another on the caller's stream)
    int profiling;
    int prof_views;                                   // views recorded and not yet read
    cudaEvent_t ev[SsbStep_kMaxProfViews][SSB_STAGE_COUNT + 1];
    int ev_ready;
    // densification outputs (off unless ssb_step_set_densify switched them on)
    int map_mode, accum_mode;
    float map_weight;
    float* accum_weight;
    float* accum_weight_den;
    int64_t* max_pairs;       // device: largest per-view pair count since it was last cleared
    float* radii;             // caller's [n] running maximum of the splats' view radii (ssb_step_set_radii), or nullptr
    int32_t sh_degree_plus1;  // active SH degree + 1, 0 = all bands (ssb_step_set_sh_degree)
    int32_t dist_tier;        // lens-distortion tier of the cameras and the rows of the next call's views (ssb_step_set_distortion)
    const float* dist_coeffs;
    // deferred backward (ssb_step_set_fused_backward): every view's aabb and screen-gradient records are kept, and the
    // projection backward of all views runs together with the optimiser, a range of splats at a time
    int def_max_views, def_count, def_last;      // def_last: slice of the last view rendered (for ssb_step_peek)
    float* def_aabb;              // [def_max_views][n][4]
    SsbScreenRec* def_vscreen;    // [def_max_views][n], zero outside a view's raster backward .. fused backward window
    float* def_grads;             // gradients of one range of splats (59 floats each, one 256-byte aligned array per attribute)
    // general loss (levels, mask, loss-map mode); off unless ssb_step_set_loss switched it on
    int loss_general;
    SsbLossConfig loss_cfg;
    int64_t loss_ws_bytes;
};

namespace ssb {

template <class T>
static int dev_alloc(T** p, int64_t count, int64_t& total) {
    int64_t bytes = align_up(count * (int64_t)sizeof(T), 256);
    if (bytes == 0) bytes = 256;
    cudaError_t e = cudaMalloc((void**)p, bytes);
    if (e != cudaSuccess) {
        *p = nullptr;
        set_error("ssb_step_create: cudaMalloc of %lld bytes failed (%s); %lld bytes already held", (long long)bytes, cudaGetErrorString(e), (long long)total);
        cudaGetLastError();
        return SSB_ERR_OUT_OF_MEMORY;
    }
    total += bytes;
    return SSB_OK;
}

static void lane_free(SsbLane& l) {
    cudaFree(l.aabb); cudaFree(l.depths); cudaFree(l.screen); cudaFree(l.v_screen);
    cudaFree(l.isect_ws); cudaFree(l.flat);
    cudaFree(l.n_isects); cudaFree(l.offsets);
    cudaFree(l.rgb); cudaFree(l.T); cudaFree(l.last_ids); cudaFree(l.v_rgb); cudaFree(l.loss_map); cudaFree(l.loss_ws); cudaFree(l.tile_live);
    if (l.stream) cudaStreamDestroy(l.stream);
    if (l.bwd_done) cudaEventDestroy(l.bwd_done);
    if (l.all_done) cudaEventDestroy(l.all_done);
}

static int lane_alloc(SsbStep* s, SsbLane& l) {
    const int64_t n = s->cfg.n_splats, P = (int64_t)s->cfg.width * s->cfg.height, cap = s->capacity;
    int64_t& tot = s->bytes;
    int e = SSB_OK;
    char* iws = nullptr;
    if (!e) e = dev_alloc(&l.aabb, n * 4, tot);
    if (!e) e = dev_alloc(&l.depths, n, tot);
    if (!e) e = dev_alloc(&l.screen, n, tot);
    if (!e) e = dev_alloc(&l.v_screen, n, tot);
    if (!e) e = dev_alloc(&iws, s->isect_ws_bytes, tot);
    l.isect_ws = iws;
    if (!e) e = dev_alloc(&l.flat, cap, tot);
    if (!e) e = dev_alloc(&l.n_isects, 1, tot);
    if (!e) e = dev_alloc(&l.offsets, (int64_t)s->tw * s->th + 1, tot);
    if (!e) e = dev_alloc(&l.rgb, P * 3, tot);
    if (!e) e = dev_alloc(&l.T, P, tot);
    if (!e) e = dev_alloc(&l.last_ids, P, tot);
    if (!e) e = dev_alloc(&l.v_rgb, P * 3, tot);
    if (e) return e;
    SSB_CUDA(cudaMemset(l.v_screen, 0, n * sizeof(SsbScreenRec)));
    SSB_CUDA(cudaMemset(l.n_isects, 0, sizeof(int64_t)));
    SSB_CUDA(cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking));
    SSB_CUDA(cudaEventCreateWithFlags(&l.bwd_done, cudaEventDisableTiming));
    SSB_CUDA(cudaEventCreateWithFlags(&l.all_done, cudaEventDisableTiming));
    return SSB_OK;
}

// All stages of one view on one stream.
static int run_view(SsbStep* s, SsbLane& l, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmats, const float* d_intrins,
                    const float* d_gt, int v, const SsbSplats* grads, int accumulate, float* d_losses, cudaStream_t st,
                    cudaEvent_t wait_before_bwd, cudaEvent_t* ev, cudaEvent_t gt_ready) {
    const int64_t n = s->cfg.n_splats;
    const int W = s->cfg.width, H = s->cfg.height;
    const int64_t P = (int64_t)W * H;
    // deferred backward: this view's aabb and gradient records go to its own slice and stay there
    const bool deferred = s->def_max_views > 0;
    float* aabb = deferred ? s->def_aabb + (int64_t)(s->def_count + v) * n * 4 : l.aabb;
    SsbScreenRec* v_screen = deferred ? s->def_vscreen + (int64_t)(s->def_count + v) * n : l.v_screen;
    SsbCameras cam{};
    cam.d_viewmats = d_viewmats + 16 * (int64_t)v;
    cam.d_intrins = d_intrins + 4 * (int64_t)v;
    cam.count = 1; cam.width = W; cam.height = H;
    cam.model = s->cfg.camera_model; cam.antialiased = s->cfg.antialiased;
    cam.distortion = s->dist_tier;
    cam.d_dist_coeffs = s->dist_coeffs ? s->dist_coeffs + 8 * (int64_t)v : nullptr;
    cam.sh_degree_plus1 = s->sh_degree_plus1;
    int e;
#define SSB_MARK(k) do { if (ev) SSB_CUDA(cudaEventRecord(ev[k], st)); } while (0)
    SSB_MARK(0);
    if ((e = ssb_project_fwd(params, shq, n, &cam, aabb, l.depths, s->radii, l.screen, st))) return e;
    SSB_MARK(1);
    // counts + scan + scatter are reported as the key stage, the per-tile sort as the sort stage;
    // the ranges come out of the scan, so that stage is empty
    // with a mask, tiles that no term of the loss reads take no pairs (src/engine/EngineTrainStep.cpp:84-126)
    const int32_t* live = nullptr;
    if (s->loss_general && s->loss_cfg.d_mask) {
        const SsbLossConfig& lc = s->loss_cfg;
        if ((e = ssb_tile_active(lc.d_mask + (int64_t)v * lc.mask_h * lc.mask_w, 1, lc.mask_h, lc.mask_w, W, H, l.tile_live, st))) return e;
        live = l.tile_live;
    }
    if ((e = launch_intersect_tiles(aabb, l.depths, l.screen, n, n, W, H, l.isect_ws, s->isect_ws_bytes, nullptr, l.flat, s->capacity,
                                 l.offsets, l.n_isects, st, ev ? ev[2] : nullptr, s->max_pairs, live))) return e;
    SSB_MARK(3);
    SSB_MARK(4);
    // the loss has no depth term, so the depth image is neither rendered nor back-propagated
    if ((e = ssb_raster_fwd(l.screen, n, l.offsets, l.flat, s->capacity, l.n_isects, 1, W, H, l.rgb, nullptr, l.T, l.last_ids, st))) return e;
    SSB_MARK(5);
    if (gt_ready) SSB_CUDA(cudaStreamWaitEvent(st, gt_ready, 0));      // the view's target image has landed
    if (s->loss_general) {
        // levels, mask and loss-map mode of ssb_step_set_loss; the view's mask lies where its target does
        SsbLossConfig lc = s->loss_cfg;
        if (lc.d_mask) lc.d_mask += (int64_t)v * lc.mask_h * lc.mask_w;
        if (!s->accum_mode) lc.loss_map_mode = 0;
        if ((e = launch_loss_multi(l.rgb, d_gt + (int64_t)v * P * 3, 1, H, W, lc, l.v_rgb, d_losses, s->accum_mode ? l.loss_map : nullptr,
                                   l.loss_ws, s->loss_ws_bytes, st))) return e;
        SSB_MARK(6);
        if (s->accum_mode && lc.loss_map_mode) {
            if ((e = ssb_raster_bwd_accum(l.screen, n, l.offsets, l.flat, s->capacity, l.n_isects, 1, W, H, nullptr, l.T, l.last_ids, l.v_rgb, nullptr,
                                          nullptr, v_screen, s->accum_mode, l.loss_map, n, nullptr, s->accum_weight, s->accum_weight_den, st))) return e;
        } else {
            if ((e = ssb_raster_bwd(l.screen, n, l.offsets, l.flat, s->capacity, l.n_isects, 1, W, H, nullptr, l.T, l.last_ids,
                                    l.v_rgb, nullptr, nullptr, v_screen, st))) return e;
        }
    } else if (s->accum_mode) {
        // the view's SSIM loss map, then the backward pass that also folds it into the per-splat weights
        SSB_CUDA(cudaMemsetAsync(l.loss_map, 0, P * sizeof(float), st));
        if ((e = launch_loss_map(l.rgb, d_gt + (int64_t)v * P * 3, 1, H, W, s->cfg.w_l1, s->cfg.w_ssim, l.v_rgb, d_losses, s->map_mode,
                                 s->map_weight, l.loss_map, st))) return e;
        SSB_MARK(6);
        if ((e = ssb_raster_bwd_accum(l.screen, n, l.offsets, l.flat, s->capacity, l.n_isects, 1, W, H, nullptr, l.T, l.last_ids, l.v_rgb, nullptr, nullptr,
                                      v_screen, s->accum_mode, l.loss_map, n, nullptr, s->accum_weight, s->accum_weight_den, st))) return e;
    } else {
        if ((e = launch_loss(l.rgb, d_gt + (int64_t)v * P * 3, 1, H, W, s->cfg.w_l1, s->cfg.w_ssim, l.v_rgb, d_losses, st))) return e;
        SSB_MARK(6);
        if ((e = ssb_raster_bwd(l.screen, n, l.offsets, l.flat, s->capacity, l.n_isects, 1, W, H, nullptr, l.T, l.last_ids,
                                l.v_rgb, nullptr, nullptr, v_screen, st))) return e;
    }
    SSB_MARK(7);
    if (!deferred) {
        if (wait_before_bwd) SSB_CUDA(cudaStreamWaitEvent(st, wait_before_bwd, 0));
        if ((e = launch_project_bwd(params, shq, n, &cam, aabb, v_screen, grads, accumulate, 1, st, nullptr, 0, -1))) return e;
    }
    SSB_MARK(8);
#undef SSB_MARK
    return SSB_OK;
}

}  // namespace ssb

extern "C" {

int ssb_step_set_loss(SsbStep* s, const SsbLossConfig* cfg) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_set_loss: NULL step");
    if (!cfg) { s->loss_general = 0; return SSB_OK; }
    if (int e = check_loss_config(cfg, "ssb_step_set_loss")) return e;
    SsbLossConfig c = *cfg;
    c.w_l1 = s->cfg.w_l1; c.w_ssim = s->cfg.w_ssim;
    const int64_t need = loss_workspace_bytes(1, s->cfg.height, s->cfg.width, c);
    const int64_t P = (int64_t)s->cfg.width * s->cfg.height;
    for (int k = 0; k < s->n_lanes; ++k) {
        SsbLane& l = s->lane[k];
        if (!l.loss_ws || s->loss_ws_bytes < need) {
            SSB_CUDA(cudaStreamSynchronize(l.stream));
            cudaFree(l.loss_ws);
            l.loss_ws = nullptr;
            char* p = nullptr;
            if (int e = dev_alloc(&p, need, s->bytes)) return e;
            l.loss_ws = p;
        }
        if (c.loss_map_mode && !l.loss_map)
            if (int e = dev_alloc(&l.loss_map, P, s->bytes)) return e;
        if (c.d_mask && !l.tile_live)
            if (int e = dev_alloc(&l.tile_live, (int64_t)s->tw * s->th, s->bytes)) return e;
    }
    s->loss_ws_bytes = std::max(s->loss_ws_bytes, need);
    s->loss_cfg = c;
    s->loss_general = 1;
    return SSB_OK;
}

int ssb_step_set_radii(SsbStep* s, float* d_radii) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_set_radii: NULL step");
    s->radii = d_radii;
    return SSB_OK;
}

int ssb_step_set_sh_degree(SsbStep* s, int32_t sh_degree) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_set_sh_degree: NULL step");
    SSB_REQUIRE(sh_degree >= 0 && sh_degree <= 3, "ssb_step_set_sh_degree: the degree must be 0..3 (got %d)", sh_degree);
    s->sh_degree_plus1 = sh_degree + 1;
    return SSB_OK;
}

int ssb_step_set_distortion(SsbStep* s, int32_t tier, const float* d_dist_coeffs) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_set_distortion: NULL step");
    const int model = s->cfg.camera_model;
    const bool built = tier == SSB_DISTORTION_NONE ||
                       ((tier == SSB_DISTORTION_OPENCV || tier == SSB_DISTORTION_THIN_PRISM) && model != SSB_CAMERA_EQUIRECT) ||
                       (tier == SSB_DISTORTION_RATIONAL && model == SSB_CAMERA_PINHOLE);
    if (!built) { set_error("ssb_step_set_distortion: unsupported camera model / distortion tier (%d, %d)", model, tier); return SSB_ERR_UNSUPPORTED; }
    s->dist_tier = tier;
    s->dist_coeffs = tier == SSB_DISTORTION_NONE ? nullptr : d_dist_coeffs;
    return SSB_OK;
}

int ssb_step_set_densify(SsbStep* s, int32_t ssim_loss_map_mode, float ssim_loss_map_weight, int32_t accum_mode,
                         float* d_accum_weight, float* d_accum_weight_den) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_set_densify: NULL step");
    SSB_REQUIRE(accum_mode >= SSB_ACCUM_NONE && accum_mode <= SSB_ACCUM_AVG, "ssb_step_set_densify: accum_mode %d is not a DensifyAccumMode", accum_mode);
    if (accum_mode == SSB_ACCUM_NONE) { s->accum_mode = 0; return SSB_OK; }
    SSB_REQUIRE(ssim_loss_map_mode >= 1 && ssim_loss_map_mode <= 3, "ssb_step_set_densify: ssim_loss_map_mode must be 1, 2 or 3 (got %d)", ssim_loss_map_mode);
    SSB_REQUIRE(d_accum_weight && (accum_mode != SSB_ACCUM_AVG || d_accum_weight_den), "ssb_step_set_densify: output array missing");
    const int64_t P = (int64_t)s->cfg.width * s->cfg.height;
    for (int k = 0; k < s->n_lanes; ++k)
        if (!s->lane[k].loss_map) {
            int e = dev_alloc(&s->lane[k].loss_map, P, s->bytes);
            if (e) return e;
        }
    s->map_mode = ssim_loss_map_mode; s->map_weight = ssim_loss_map_weight; s->accum_mode = accum_mode;
    s->accum_weight = d_accum_weight; s->accum_weight_den = d_accum_weight_den;
    return SSB_OK;
}

void ssb_step_destroy(SsbStep* s) {
    if (!s) return;
    for (int k = 0; k < SsbStep_kLanes; ++k) ssb::lane_free(s->lane[k]);
    if (s->fork) cudaEventDestroy(s->fork);
    cudaFree(s->max_pairs);
    cudaFree(s->def_aabb); cudaFree(s->def_vscreen); cudaFree(s->def_grads);
    if (s->ev_ready)
        for (int v = 0; v < SsbStep_kMaxProfViews; ++v)
            for (int k = 0; k <= SSB_STAGE_COUNT; ++k) cudaEventDestroy(s->ev[v][k]);
    delete s;
}

int ssb_step_create(const SsbStepConfig* cfg, SsbStep** out) {
    using namespace ssb;
    SSB_REQUIRE(cfg && out, "ssb_step_create: NULL argument");
    SSB_REQUIRE(cfg->n_splats > 0 && cfg->width > 0 && cfg->height > 0, "ssb_step_create: bad sizes");
    SSB_REQUIRE(cfg->n_splats < ((int64_t)1 << 31), "ssb_step_create: splat count must fit int32");
    if (cfg->camera_model < SSB_CAMERA_PINHOLE || cfg->camera_model > SSB_CAMERA_EQUIRECT) {
        set_error("ssb_step_create: camera model %d not supported", cfg->camera_model); return SSB_ERR_UNSUPPORTED;
    }
    SsbStep* s = new (std::nothrow) SsbStep();
    SSB_REQUIRE(s != nullptr, "ssb_step_create: out of host memory");
    memset(s, 0, sizeof(*s));
    s->cfg = *cfg;
    s->tw = (cfg->width + kTile - 1) / kTile;
    s->th = (cfg->height + kTile - 1) / kTile;
    s->capacity = cfg->isect_capacity > 0 ? cfg->isect_capacity : 12 * cfg->n_splats;
    if (s->capacity >= ((int64_t)1 << 30)) s->capacity = ((int64_t)1 << 30) - 1;
    s->isect_ws_bytes = ssb_intersect_tiles_workspace_bytes((int64_t)s->tw * s->th, s->capacity);
    s->n_lanes = SsbStep_kLanes;
    for (int k = 0; k < s->n_lanes; ++k) {
        int e = lane_alloc(s, s->lane[k]);
        if (e) { ssb_step_destroy(s); return e; }
    }
    {
        int e = dev_alloc(&s->max_pairs, 1, s->bytes);
        if (!e) e = check_cuda(cudaMemset(s->max_pairs, 0, sizeof(int64_t)), "ssb_step_create: cudaMemset");
        if (e) { ssb_step_destroy(s); return e; }
    }
    cudaError_t ce = cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming);
    if (ce != cudaSuccess) { ssb_step_destroy(s); return check_cuda(ce, "ssb_step_create: cudaEventCreate"); }
    *out = s;
    return SSB_OK;
}

int64_t ssb_step_device_bytes(const SsbStep* step) { return step ? step->bytes : 0; }

int ssb_step_views(SsbStep* s, const SsbSplats* params, const SsbShQuant* shq,
                   const float* d_viewmats, const float* d_intrins, const float* d_gt, int32_t n_views,
                   const SsbSplats* grads, int accumulate, float* d_losses, void* stream) {
    return ssb_step_views_gated(s, params, shq, d_viewmats, d_intrins, d_gt, n_views, nullptr, grads, accumulate, d_losses, stream);
}

int ssb_step_views_gated(SsbStep* s, const SsbSplats* params, const SsbShQuant* shq,
                         const float* d_viewmats, const float* d_intrins, const float* d_gt, int32_t n_views,
                         void* const* gt_ready, const SsbSplats* grads, int accumulate, float* d_losses, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(s && params && d_viewmats && d_intrins && d_gt && grads, "ssb_step_views: NULL argument");
    SSB_REQUIRE(n_views >= 0, "ssb_step_views: bad view count");
    SSB_REQUIRE(s->def_max_views == 0 || s->def_count + n_views <= s->def_max_views, "ssb_step_views: %d views kept + %d new exceed the room for %d "
                "(ssb_step_set_fused_backward)", s->def_count, n_views, s->def_max_views);
    cudaStream_t user = (cudaStream_t)stream;
    if (n_views == 0) return SSB_OK;
    if (s->profiling || n_views == 1) {
        // one view, or timing requested: everything on the caller's stream, in order
        for (int v = 0; v < n_views; ++v) {
            const bool prof = s->profiling && s->prof_views < SsbStep_kMaxProfViews;
            int e = run_view(s, s->lane[0], params, shq, d_viewmats, d_intrins, d_gt, v, grads, (accumulate || v > 0) ? 1 : 0, d_losses, user,
                             nullptr, prof ? s->ev[s->prof_views] : nullptr, gt_ready ? (cudaEvent_t)gt_ready[v] : nullptr);
            if (e) return e;
            if (prof) s->prof_views++;
        }
        s->last_lane = 0;
        if (s->def_max_views > 0) { s->def_count += n_views; s->def_last = s->def_count - 1; }
        return SSB_OK;
    }
    SSB_CUDA(cudaEventRecord(s->fork, user));
    for (int k = 0; k < s->n_lanes; ++k) SSB_CUDA(cudaStreamWaitEvent(s->lane[k].stream, s->fork, 0));
    cudaEvent_t prev_bwd = nullptr;
    for (int v = 0; v < n_views; ++v) {
        SsbLane& l = s->lane[v % s->n_lanes];
        int e = run_view(s, l, params, shq, d_viewmats, d_intrins, d_gt, v, grads, (accumulate || v > 0) ? 1 : 0, d_losses, l.stream, prev_bwd, nullptr,
                         gt_ready ? (cudaEvent_t)gt_ready[v] : nullptr);
        if (e) return e;
        SSB_CUDA(cudaEventRecord(l.bwd_done, l.stream));
        prev_bwd = l.bwd_done;
        s->last_lane = v % s->n_lanes;
    }
    for (int k = 0; k < s->n_lanes; ++k) {
        SSB_CUDA(cudaEventRecord(s->lane[k].all_done, s->lane[k].stream));
        SSB_CUDA(cudaStreamWaitEvent(user, s->lane[k].all_done, 0));
    }
    if (s->def_max_views > 0) { s->def_count += n_views; s->def_last = s->def_count - 1; }
    return SSB_OK;
}

// Splats per range of the fused backward: the range's 59 gradient floats (31 MB) are written by one kernel and read by the
// next, and stay in the 126 MB L2 in between together with the records that stream through.  Ranges alternate between the
// step's two streams, each with its own scratch, so that one range's optimiser kernels run beside the next range's
// projection backward (a range alone is less than four waves of CTAs).
static const int64_t kFusedRange = 131072;

int ssb_step_set_fused_backward(SsbStep* s, int32_t max_views) {
    using namespace ssb;
    SSB_REQUIRE(s && max_views >= 0, "ssb_step_set_fused_backward: bad argument");
    const int64_t n = s->cfg.n_splats;
    if (max_views > s->def_max_views) {
        for (int k = 0; k < s->n_lanes; ++k) SSB_CUDA(cudaStreamSynchronize(s->lane[k].stream));
        cudaFree(s->def_aabb); cudaFree(s->def_vscreen);
        s->def_aabb = nullptr; s->def_vscreen = nullptr;
        if (int e = dev_alloc(&s->def_aabb, (int64_t)max_views * n * 4, s->bytes)) return e;
        if (int e = dev_alloc(&s->def_vscreen, (int64_t)max_views * n, s->bytes)) return e;
        SSB_CUDA(cudaMemset(s->def_vscreen, 0, (size_t)max_views * n * sizeof(SsbScreenRec)));
        if (!s->def_grads)
            if (int e = dev_alloc(&s->def_grads, SsbStep_kLanes * (6 * 64 + std::min(kFusedRange, align_up(n, 256)) * 59), s->bytes)) return e;
    }
    s->def_max_views = max_views;      // 0: back to one projection backward per view (the buffers are kept)
    s->def_count = 0;
    return SSB_OK;
}

}  // extern "C"

namespace ssb {

// One range of splats of the fused backward + optimiser pass: the projection backward of all views writes the range's 59
// gradient floats per splat into `scratch` (which stays in L2), the optimiser kernels read them from there.
static int fused_backward_range(const SsbSplats* params, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                                SsbScreenRec* d_v_screen, int clear_v_screen, const SsbMomentsQ16* nq, const SsbSplats* m1, const SsbSplats* m2,
                                const SsbShAdamState* sh_state, const SsbAdamConfig* c, const SsbAdamExtras* extras, float* scratch, int64_t range,
                                int64_t first, int64_t count, void* stream) {
    // the range's gradient arrays, each on a 256-byte boundary
    float* g_means = scratch;
    float* g_quats = g_means + align_up(3 * range, 64);
    float* g_scales = g_quats + align_up(4 * range, 64);
    float* g_opac = g_scales + align_up(3 * range, 64);
    float* g_dc = g_opac + align_up(range, 64);
    float* g_sh = g_dc + align_up(3 * range, 64);
    // pointers moved back by the range's start: kernels index gradients by the splat's own number
    SsbSplats g;
    g.means = g_means - 3 * first; g.quats = g_quats - 4 * first; g.scales = g_scales - 3 * first; g.opacities = g_opac - first;
    g.features_dc = g_dc - 3 * first; g.features_sh = g_sh - 45 * first;
    if (int e = launch_project_bwd(params, shq, n, cams, d_aabb, d_v_screen, &g, 0, clear_v_screen, stream, nullptr, first, count)) return e;
    SsbSplats ga = g;
    if (sh_state) ga.features_sh = nullptr;      // the SH update is the quantised one below
    if (nq) {
        // Moments of the five non-SH arrays in 16-bit codes.  The fused kernel of the reference scales the DC regulariser like the
        // SH one, 2 w / (3 n) (src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:1137, :355-358), where its unfused kernel with
        // these moments takes w as it is; ssb_adam_step_q16 follows the unfused kernel, so the scaled weight is handed to it.
        SsbAdamConfig cq = *c;
        cq.sh_reg_weight = 2.0f * c->sh_reg_weight / (float)(3 * n);
        if (int e = ssb_adam_step_q16(params, &ga, nq, first, count, &cq, extras, stream)) return e;
        if (!sh_state) {
            // fp32 SH: fused_adam_step's decay is 2 l2 / numel of the call, so l2 is scaled to the range's share of the array
            const int64_t off = 45 * first, numel = 45 * count;
            if (int e = ssb_adam_plain(params->features_sh + off, g.features_sh + off, m1->features_sh + off, m2->features_sh + off, numel, 45,
                                       c->lr_features_sh, c->step, extras && extras->d_steps ? extras->d_steps + first : nullptr,
                                       c->sh_reg_weight * (float)count / (float)n, 0.0f, c->grad_scale, 0, stream)) return e;
        }
    } else {
        SsbSplats p = *params, a1 = *m1, a2 = *m2;
        if (sh_state) { p.features_sh = nullptr; a1.features_sh = nullptr; a2.features_sh = nullptr; }
        if (int e = ssb_adam_step_ex(&p, &ga, &a1, &a2, first, count, c, extras, stream)) return e;
    }
    if (sh_state && sh_state->layout == SSB_SH_LAYOUT_SPLAT_BLOCKS) {
        // the reference's own layout for this path: bounds per 256 splats; a range is a whole number of such blocks
        if (int e = ssb_adam_step_sh_splat_blocks(g.features_sh, sh_state->d_optim_packed, sh_state->d_optim_bounds, sh_state->d_value_packed,
                                                  sh_state->d_value_bounds, sh_state->value_bits, first, count, n, cams->sh_degree_plus1, c,
                                                  extras ? extras->d_steps : nullptr, stream)) return e;
    } else if (sh_state) {
        void* values = sh_state->value_bits == 32 ? (void*)params->features_sh : sh_state->d_value_packed;
        if (int e = ssb_adam_step_sh_quantized_ex(g.features_sh, sh_state->d_optim_packed, sh_state->d_optim_bounds, values, sh_state->d_value_bounds,
                                                  sh_state->value_bits, sh_state->optim_bits ? sh_state->optim_bits : 8, first * 45, count * 45, n * 45,
                                                  c, extras ? extras->d_steps : nullptr, 45, stream)) return e;
    }
    return SSB_OK;
}

static int64_t fused_scratch_floats(int64_t n) { return 6 * 64 + std::min(kFusedRange, align_up(n, 256)) * 59; }

}  // namespace ssb

extern "C" {

int64_t ssb_project_bwd_optimize_workspace_bytes(int64_t n) { return n < 0 ? SSB_ERR_INVALID_ARGUMENT : ssb::fused_scratch_floats(n) * (int64_t)sizeof(float); }

static int project_bwd_optimize_impl(const SsbSplats* params, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                                     const SsbScreenRec* d_v_screen, const SsbMomentsQ16* nq, const SsbSplats* m1, const SsbSplats* m2,
                                     const SsbShAdamState* sh_state, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* d_workspace,
                                     int64_t workspace_bytes, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(params && cams && d_aabb && d_v_screen && cfg && d_workspace, "ssb_project_bwd_optimize: NULL argument");
    SSB_REQUIRE(nq ? (sh_state || (m1 && m2 && m1->features_sh && m2->features_sh)) : (m1 && m2),
                "ssb_project_bwd_optimize: moments missing (with 16-bit moments m1 / m2 carry features_sh, unless the SH state is quantised)");
    SSB_REQUIRE(n >= 0 && cams->count >= 0, "ssb_project_bwd_optimize: bad sizes");
    SSB_REQUIRE(workspace_bytes >= ssb_project_bwd_optimize_workspace_bytes(n), "ssb_project_bwd_optimize: workspace too small");
    SSB_REQUIRE(((uintptr_t)d_workspace & 255) == 0, "ssb_project_bwd_optimize: the workspace must be 256-byte aligned");
    SSB_REQUIRE(!sh_state || params->features_sh == nullptr || sh_state->value_bits == 32,
                "ssb_project_bwd_optimize: SH values are either plain (params->features_sh) or quantised (sh_state), not both");
    if (n == 0 || cams->count == 0) return SSB_OK;
    SsbAdamConfig c = *cfg;
    c.zero_grad = 0;
    const int64_t range = std::min(kFusedRange, align_up(n, 256));
    for (int64_t first = 0; first < n; first += range) {
        if (int e = fused_backward_range(params, shq, n, cams, d_aabb, const_cast<SsbScreenRec*>(d_v_screen), 0, nq, m1, m2, sh_state, &c, extras,
                                         (float*)d_workspace, range, first, std::min(range, n - first), stream)) return e;
    }
    return SSB_OK;
}

int ssb_project_bwd_optimize(const SsbSplats* params, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                             const SsbScreenRec* d_v_screen, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                             const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* d_workspace, int64_t workspace_bytes, void* stream) {
    return project_bwd_optimize_impl(params, shq, n, cams, d_aabb, d_v_screen, nullptr, m1, m2, sh_state, cfg, extras, d_workspace, workspace_bytes, stream);
}

int ssb_project_bwd_optimize_q16(const SsbSplats* params, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                                 const SsbScreenRec* d_v_screen, const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2,
                                 const SsbShAdamState* sh_state, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* d_workspace,
                                 int64_t workspace_bytes, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(moments, "ssb_project_bwd_optimize_q16: NULL moments");
    return project_bwd_optimize_impl(params, shq, n, cams, d_aabb, d_v_screen, moments, m1, m2, sh_state, cfg, extras, d_workspace, workspace_bytes, stream);
}

static int step_backward_optimize_impl(SsbStep* s, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmats, const float* d_intrins,
                                       int32_t n_views, const SsbMomentsQ16* nq, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state,
                                       const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(s && params && d_viewmats && d_intrins && cfg, "ssb_step_backward_optimize: NULL argument");
    SSB_REQUIRE(nq ? (sh_state || (m1 && m2 && m1->features_sh && m2->features_sh)) : (m1 && m2),
                "ssb_step_backward_optimize: moments missing (with 16-bit moments m1 / m2 carry features_sh, unless the SH state is quantised)");
    SSB_REQUIRE(s->def_max_views > 0, "ssb_step_backward_optimize: the step does not keep its views (ssb_step_set_fused_backward)");
    SSB_REQUIRE(n_views == s->def_count && n_views <= s->def_max_views, "ssb_step_backward_optimize: %d views given, %d kept (room for %d)", n_views,
                s->def_count, s->def_max_views);
    SSB_REQUIRE(!sh_state || params->features_sh == nullptr || sh_state->value_bits == 32,
                "ssb_step_backward_optimize: SH values are either plain (params->features_sh) or quantised (sh_state), not both");
    const int64_t n = s->cfg.n_splats;
    s->def_count = 0;
    if (n_views == 0) return SSB_OK;
    SsbCameras cams{};
    cams.d_viewmats = d_viewmats; cams.d_intrins = d_intrins; cams.count = n_views;
    cams.width = s->cfg.width; cams.height = s->cfg.height; cams.model = s->cfg.camera_model; cams.antialiased = s->cfg.antialiased;
    cams.distortion = s->dist_tier; cams.d_dist_coeffs = s->dist_coeffs; cams.sh_degree_plus1 = s->sh_degree_plus1;
    const int64_t range = std::min(kFusedRange, align_up(n, 256));
    const int64_t scratch_floats = fused_scratch_floats(n);
    SsbAdamConfig c = *cfg;
    c.zero_grad = 0;                       // every range overwrites the scratch
    cudaStream_t user = (cudaStream_t)stream;
    const bool two = n > range;            // more than one range: alternate between the lanes' streams
    if (two) {
        SSB_CUDA(cudaEventRecord(s->fork, user));
        for (int k = 0; k < s->n_lanes; ++k) SSB_CUDA(cudaStreamWaitEvent(s->lane[k].stream, s->fork, 0));
    }
    int turn = 0;
    for (int64_t first = 0; first < n; first += range, ++turn) {
        void* range_stream = two ? (void*)s->lane[turn % s->n_lanes].stream : (void*)user;
        float* scratch = s->def_grads + (two ? turn % s->n_lanes : 0) * scratch_floats;
        if (int e = fused_backward_range(params, shq, n, &cams, s->def_aabb, s->def_vscreen, 1, nq, m1, m2, sh_state, &c, extras, scratch, range, first,
                                         std::min(range, n - first), range_stream)) return e;
    }
    if (two)
        for (int k = 0; k < s->n_lanes; ++k) {
            SSB_CUDA(cudaEventRecord(s->lane[k].all_done, s->lane[k].stream));
            SSB_CUDA(cudaStreamWaitEvent(user, s->lane[k].all_done, 0));
        }
    return SSB_OK;
}

int ssb_step_backward_optimize(SsbStep* s, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmats, const float* d_intrins,
                               int32_t n_views, const SsbSplats* m1, const SsbSplats* m2, const SsbShAdamState* sh_state, const SsbAdamConfig* cfg,
                               const SsbAdamExtras* extras, void* stream) {
    return step_backward_optimize_impl(s, params, shq, d_viewmats, d_intrins, n_views, nullptr, m1, m2, sh_state, cfg, extras, stream);
}

int ssb_step_backward_optimize_q16(SsbStep* s, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmats, const float* d_intrins,
                                   int32_t n_views, const SsbMomentsQ16* moments, const SsbSplats* m1, const SsbSplats* m2,
                                   const SsbShAdamState* sh_state, const SsbAdamConfig* cfg, const SsbAdamExtras* extras, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(moments, "ssb_step_backward_optimize_q16: NULL moments");
    return step_backward_optimize_impl(s, params, shq, d_viewmats, d_intrins, n_views, moments, m1, m2, sh_state, cfg, extras, stream);
}

int ssb_step_set_profiling(SsbStep* s, int enable) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_set_profiling: NULL step");
    if (enable && !s->ev_ready) {
        for (int v = 0; v < SsbStep_kMaxProfViews; ++v)
            for (int k = 0; k <= SSB_STAGE_COUNT; ++k) SSB_CUDA(cudaEventCreate(&s->ev[v][k]));
        s->ev_ready = 1;
    }
    s->profiling = enable ? 1 : 0;
    s->prof_views = 0;
    return SSB_OK;
}

int ssb_step_get_profile(SsbStep* s, float* ms, int32_t* n_views) {
    using namespace ssb;
    SSB_REQUIRE(s && ms && n_views, "ssb_step_get_profile: NULL argument");
    *n_views = s->prof_views;
    for (int v = 0; v < s->prof_views; ++v) {
        SSB_CUDA(cudaEventSynchronize(s->ev[v][SSB_STAGE_COUNT]));
        for (int k = 0; k < SSB_STAGE_COUNT; ++k) {
            float t = 0.f;
            SSB_CUDA(cudaEventElapsedTime(&t, s->ev[v][k], s->ev[v][k + 1]));
            ms[k] += t;
        }
    }
    s->prof_views = 0;
    return SSB_OK;
}

int ssb_step_last_isects(SsbStep* s, int64_t* h_n_isects, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(s && h_n_isects, "ssb_step_last_isects: NULL argument");
    SsbLane& l = s->lane[s->last_lane];
    SSB_CUDA(cudaMemcpyAsync(h_n_isects, l.n_isects, sizeof(int64_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SSB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (*h_n_isects > s->capacity) {
        set_error("ssb_step: %lld (splat, tile) pairs exceed the capacity of %lld; pairs beyond it were dropped", (long long)*h_n_isects, (long long)s->capacity);
        return SSB_ERR_CAPACITY;
    }
    return SSB_OK;
}

const int64_t* ssb_step_max_pairs_device(const SsbStep* s) { return s ? s->max_pairs : nullptr; }

int64_t ssb_step_isect_capacity(const SsbStep* s) { return s ? s->capacity : 0; }

int ssb_step_status(SsbStep* s, int64_t* h_max_pairs, int reset, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_status: NULL step");
    cudaStream_t st = (cudaStream_t)stream;
    int64_t m = 0;
    SSB_CUDA(cudaMemcpyAsync(&m, s->max_pairs, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
    if (reset) SSB_CUDA(cudaMemsetAsync(s->max_pairs, 0, sizeof(int64_t), st));
    SSB_CUDA(cudaStreamSynchronize(st));
    if (h_max_pairs) *h_max_pairs = m;
    if (m > s->capacity) {
        set_error("ssb_step: a view had %lld (splat, tile) pairs, more than the capacity of %lld; the pairs beyond it were dropped "
                  "(create the step with a larger isect_capacity)", (long long)m, (long long)s->capacity);
        return SSB_ERR_CAPACITY;
    }
    return SSB_OK;
}

int ssb_step_render(SsbStep* s, const SsbSplats* params, const SsbShQuant* shq, const float* d_viewmat, const float* d_intrin,
                    float* d_rgb, float* d_depth, float* d_T, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(s && params && d_viewmat && d_intrin && d_rgb, "ssb_step_render: NULL argument");
    const int64_t n = s->cfg.n_splats;
    const int W = s->cfg.width, H = s->cfg.height;
    const int64_t P = (int64_t)W * H;
    SsbLane& l = s->lane[0];
    cudaStream_t st = (cudaStream_t)stream;
    // the lane's buffers may still be in use by views enqueued on the lane's own stream
    SSB_CUDA(cudaEventRecord(l.all_done, l.stream));
    SSB_CUDA(cudaStreamWaitEvent(st, l.all_done, 0));
    SsbCameras cam{};
    cam.d_viewmats = d_viewmat; cam.d_intrins = d_intrin; cam.count = 1; cam.width = W; cam.height = H;
    cam.model = s->cfg.camera_model; cam.antialiased = s->cfg.antialiased;
    cam.distortion = s->dist_tier; cam.d_dist_coeffs = s->dist_coeffs; cam.sh_degree_plus1 = s->sh_degree_plus1;
    int e;
    if ((e = ssb_project_fwd(params, shq, n, &cam, l.aabb, l.depths, nullptr, l.screen, st))) return e;
    if ((e = launch_intersect_tiles(l.aabb, l.depths, l.screen, n, n, W, H, l.isect_ws, s->isect_ws_bytes, nullptr, l.flat, s->capacity,
                                 l.offsets, l.n_isects, st, nullptr, s->max_pairs, nullptr))) return e;
    // T and the last-blended indices are by-products the caller may not want: they land in the lane's own images
    if ((e = ssb_raster_fwd(l.screen, n, l.offsets, l.flat, s->capacity, l.n_isects, 1, W, H, d_rgb, d_depth, d_T ? d_T : l.T, l.last_ids, st))) return e;
    // later views on the lane wait for this render to be done with its buffers
    SSB_CUDA(cudaEventRecord(l.all_done, st));
    SSB_CUDA(cudaStreamWaitEvent(l.stream, l.all_done, 0));
    s->last_lane = 0;
    (void)P;
    return SSB_OK;
}

int ssb_step_peek(SsbStep* s, const float** d_rgb, const float** d_depth, const float** d_T,
                  const int32_t** d_last_ids, const SsbScreenRec** d_screen, const float** d_aabb) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_peek: NULL step");
    SsbLane& l = s->lane[s->last_lane];
    if (d_rgb) *d_rgb = l.rgb;
    if (d_depth) *d_depth = nullptr;      // the step renders no depth image (its loss has no depth term)
    if (d_T) *d_T = l.T;
    if (d_last_ids) *d_last_ids = l.last_ids;
    if (d_screen) *d_screen = l.screen;
    if (d_aabb) *d_aabb = s->def_max_views > 0 ? s->def_aabb + (int64_t)s->def_last * s->cfg.n_splats * 4 : l.aabb;
    return SSB_OK;
}

}  // extern "C"
