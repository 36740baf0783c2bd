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
#include "ssb_common.cuh"

#include <new>

enum { SsbStep_kMaxProfViews = 64 };

struct SsbStep {
    SsbStepConfig cfg;
    int tw, th;
    int64_t capacity;
    int64_t bytes;
    // per-view intermediates
    float* aabb;          // [n][4]
    float* depths;        // [n]
    float* radii;         // [n]
    SsbScreenRec* screen; // [n]
    SsbScreenRec* v_screen;
    void* keys_ws; int64_t keys_ws_bytes;
    void* sort_ws; int64_t sort_ws_bytes;
    int64_t* ids[2];
    int32_t* flat[2];
    int64_t* n_isects;    // device
    int32_t* offsets;     // [tiles]
    float* rgb; float* depth; float* T; int32_t* last_ids; float* v_rgb;
    int sel;
    // optional per-stage timing
    int profiling;
    int prof_views;                                   // views recorded and not yet read
    cudaEvent_t ev[SsbStep_kMaxProfViews][SSB_STAGE_COUNT + 1];
    int ev_ready;
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

}  // namespace ssb

extern "C" {

void ssb_step_destroy(SsbStep* s) {
    if (!s) return;
    cudaFree(s->aabb); cudaFree(s->depths); cudaFree(s->radii); cudaFree(s->screen); cudaFree(s->v_screen);
    cudaFree(s->keys_ws); cudaFree(s->sort_ws);
    cudaFree(s->ids[0]); cudaFree(s->ids[1]); cudaFree(s->flat[0]); cudaFree(s->flat[1]);
    cudaFree(s->n_isects); cudaFree(s->offsets);
    cudaFree(s->rgb); cudaFree(s->depth); cudaFree(s->T); cudaFree(s->last_ids); cudaFree(s->v_rgb);
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
    if (cfg->camera_model != SSB_CAMERA_PINHOLE) { set_error("ssb_step_create: camera model %d not supported", cfg->camera_model); return SSB_ERR_UNSUPPORTED; }
    SsbStep* s = new (std::nothrow) SsbStep();
    SSB_REQUIRE(s != nullptr, "ssb_step_create: out of host memory");
    memset(s, 0, sizeof(*s));
    s->cfg = *cfg;
    s->tw = (cfg->width + kTile - 1) / kTile;
    s->th = (cfg->height + kTile - 1) / kTile;
    s->capacity = cfg->isect_capacity > 0 ? cfg->isect_capacity : 12 * cfg->n_splats;
    if (s->capacity >= ((int64_t)1 << 30)) s->capacity = ((int64_t)1 << 30) - 1;
    const int64_t n = cfg->n_splats, P = (int64_t)cfg->width * cfg->height, cap = s->capacity;
    s->keys_ws_bytes = ssb_tile_keys_workspace_bytes(n);
    s->sort_ws_bytes = ssb_sort_workspace_bytes(cap);
    int e = SSB_OK;
    int64_t& tot = s->bytes;
    char* kws = nullptr; char* sws = nullptr;
    if (!e) e = dev_alloc(&s->aabb, n * 4, tot);
    if (!e) e = dev_alloc(&s->depths, n, tot);
    if (!e) e = dev_alloc(&s->radii, n, tot);
    if (!e) e = dev_alloc(&s->screen, n, tot);
    if (!e) e = dev_alloc(&s->v_screen, n, tot);
    if (!e) e = dev_alloc(&kws, s->keys_ws_bytes, tot);
    if (!e) e = dev_alloc(&sws, s->sort_ws_bytes, tot);
    s->keys_ws = kws; s->sort_ws = sws;
    for (int k = 0; k < 2 && !e; ++k) {
        e = dev_alloc(&s->ids[k], cap, tot);
        if (!e) e = dev_alloc(&s->flat[k], cap, tot);
    }
    if (!e) e = dev_alloc(&s->n_isects, 1, tot);
    if (!e) e = dev_alloc(&s->offsets, (int64_t)s->tw * s->th + 1, tot);
    if (!e) e = dev_alloc(&s->rgb, P * 3, tot);
    if (!e) e = dev_alloc(&s->depth, P, tot);
    if (!e) e = dev_alloc(&s->T, P, tot);
    if (!e) e = dev_alloc(&s->last_ids, P, tot);
    if (!e) e = dev_alloc(&s->v_rgb, P * 3, tot);
    if (e) { ssb_step_destroy(s); return e; }
    cudaError_t ce = cudaMemset(s->v_screen, 0, n * sizeof(SsbScreenRec));
    if (ce == cudaSuccess) ce = cudaMemset(s->radii, 0, n * sizeof(float));
    if (ce == cudaSuccess) ce = cudaMemset(s->n_isects, 0, sizeof(int64_t));
    if (ce != cudaSuccess) { ssb_step_destroy(s); return check_cuda(ce, "ssb_step_create: cudaMemset"); }
    *out = s;
    return SSB_OK;
}

int64_t ssb_step_device_bytes(const SsbStep* step) { return step ? step->bytes : 0; }

int ssb_step_views(SsbStep* s, const SsbSplats* params, const SsbShQuant* shq,
                   const float* d_viewmats, const float* d_intrins, const float* d_gt, int32_t n_views,
                   const SsbSplats* grads, int accumulate, float* d_losses, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(s && params && d_viewmats && d_intrins && d_gt && grads, "ssb_step_views: NULL argument");
    SSB_REQUIRE(n_views >= 0, "ssb_step_views: bad view count");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t n = s->cfg.n_splats;
    const int W = s->cfg.width, H = s->cfg.height;
    const int64_t P = (int64_t)W * H;
    const int64_t n_tiles = (int64_t)s->tw * s->th;
    const int end_bit = 32 + ssb_tile_n_bits(n_tiles);
    for (int v = 0; v < n_views; ++v) {
        SsbCameras cam;
        cam.d_viewmats = d_viewmats + 16 * (int64_t)v;
        cam.d_intrins = d_intrins + 4 * (int64_t)v;
        cam.count = 1; cam.width = W; cam.height = H;
        cam.model = s->cfg.camera_model; cam.antialiased = s->cfg.antialiased;
        int e;
        const bool prof = s->profiling && s->prof_views < SsbStep_kMaxProfViews;
        cudaEvent_t* ev = prof ? s->ev[s->prof_views] : nullptr;
#define SSB_MARK(k) do { if (prof) SSB_CUDA(cudaEventRecord(ev[k], st)); } while (0)
        SSB_MARK(0);
        if ((e = ssb_project_fwd(params, shq, n, &cam, s->aabb, s->depths, nullptr, s->screen, st))) return e;
        SSB_MARK(1);
        if ((e = ssb_tile_keys(s->aabb, s->depths, s->screen, n, n, W, H, s->keys_ws, s->keys_ws_bytes, nullptr, nullptr,
                               s->ids[0], s->flat[0], s->capacity, s->n_isects, nullptr, st))) return e;
        SSB_MARK(2);
        int32_t sel = 0;
        if ((e = ssb_sort_pairs_u64(s->ids[0], s->flat[0], s->ids[1], s->flat[1], s->n_isects, s->capacity, 0, end_bit,
                                    s->sort_ws, s->sort_ws_bytes, &sel, st))) return e;
        s->sel = sel;
        SSB_MARK(3);
        if ((e = ssb_tile_ranges(s->ids[sel], s->n_isects, s->capacity, n_tiles, s->offsets, st))) return e;
        SSB_MARK(4);
        if ((e = ssb_raster_fwd(s->screen, s->offsets, s->flat[sel], s->n_isects, 1, W, H, s->rgb, s->depth, s->T, s->last_ids, st))) return e;
        SSB_MARK(5);
        if ((e = launch_loss(s->rgb, d_gt + (int64_t)v * P * 3, 1, H, W, s->cfg.w_l1, s->cfg.w_ssim, s->v_rgb, d_losses, st))) return e;
        SSB_MARK(6);
        if ((e = ssb_raster_bwd(s->screen, s->offsets, s->flat[sel], s->n_isects, 1, W, H, s->depth, s->T, s->last_ids,
                                s->v_rgb, nullptr, nullptr, s->v_screen, st))) return e;
        SSB_MARK(7);
        if ((e = launch_project_bwd(params, shq, n, &cam, s->aabb, s->v_screen, grads, (accumulate || v > 0) ? 1 : 0, 1, st))) return e;
        SSB_MARK(8);
#undef SSB_MARK
        if (prof) s->prof_views++;
    }
    return SSB_OK;
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
    SSB_CUDA(cudaMemcpyAsync(h_n_isects, s->n_isects, sizeof(int64_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SSB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    int e = ssb_sort_check(s->sort_ws, stream);
    if (e) return e;
    if (*h_n_isects > s->capacity) {
        set_error("ssb_step: %lld (splat, tile) pairs exceed the capacity of %lld; pairs beyond it were dropped", (long long)*h_n_isects, (long long)s->capacity);
        return SSB_ERR_CAPACITY;
    }
    return SSB_OK;
}

int ssb_step_peek(SsbStep* s, const float** d_rgb, const float** d_depth, const float** d_T,
                  const int32_t** d_last_ids, const SsbScreenRec** d_screen, const float** d_aabb) {
    using namespace ssb;
    SSB_REQUIRE(s, "ssb_step_peek: NULL step");
    if (d_rgb) *d_rgb = s->rgb;
    if (d_depth) *d_depth = s->depth;
    if (d_T) *d_T = s->T;
    if (d_last_ids) *d_last_ids = s->last_ids;
    if (d_screen) *d_screen = s->screen;
    if (d_aabb) *d_aabb = s->aabb;
    return SSB_OK;
}

}  // extern "C"
