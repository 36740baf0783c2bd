// Shared definitions for the kernels of libssb_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <math.h>

#include "../../include/ssb.h"

namespace ssb {

constexpr float kAlphaThreshold = 1.0f / 255.0f;
constexpr int kTile = SSB_TILE;
constexpr int kNumSh = SSB_NUM_SH;
constexpr float kShC0 = 0.2820947917738781f;

// Thread-local error text and the process-wide launch counter.
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
int check_cuda(cudaError_t e, const char* what);
// Opts `kernel` in to `bytes` of dynamic shared memory on the current device (once per kernel and device).
int ensure_dynamic_smem(const void* kernel, int bytes);
constexpr int kMaxDevices = 64;
// Device address of the current device's sticky status word (SSB_STATUS_* bits), or nullptr.
unsigned int* device_status_word();

#define SSB_REQUIRE(cond, ...)                      \
    do {                                            \
        if (!(cond)) {                              \
            ::ssb::set_error(__VA_ARGS__);          \
            return SSB_ERR_INVALID_ARGUMENT;        \
        }                                           \
    } while (0)

#define SSB_CUDA(expr)                                              \
    do {                                                            \
        int _e = ::ssb::check_cuda((expr), #expr);                  \
        if (_e != SSB_OK) return _e;                                \
    } while (0)

// Call after every kernel launch: counts it and turns a launch error into a status.
#define SSB_LAUNCHED(name)                                          \
    do {                                                            \
        ::ssb::count_launch();                                      \
        int _e = ::ssb::check_cuda(cudaGetLastError(), name);       \
        if (_e != SSB_OK) return _e;                                \
    } while (0)

// launchers shared between translation units
int launch_loss(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                float* d_v_render, float* d_losses, cudaStream_t st);
int launch_loss_map(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                    float* d_v_render, float* d_losses, int map_mode, float map_weight, float* d_loss_map, cudaStream_t st);
int64_t loss_workspace_bytes(int B, int H, int W, const SsbLossConfig& cfg);
int launch_loss_multi(const float* d_render, const float* d_gt, int B, int H, int W, const SsbLossConfig& cfg, float* d_v_render,
                      float* d_losses, float* d_loss_map, void* d_ws, int64_t ws_bytes, cudaStream_t st);
int check_loss_config(const SsbLossConfig* cfg, const char* who);
int launch_project_bwd(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                       SsbScreenRec* d_v_screen, const SsbSplats* grads, int accumulate, int clear_v_screen, void* stream,
                       const int32_t* d_pair_of, int64_t range_first, int64_t range_count);
int launch_project_fwd_pack_pass(int pass, const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams,
                                 int32_t* d_flags, float* d_aabb, float* d_depths, float* d_radii, SsbScreenRec* d_screen,
                                 int32_t* d_camera_ids, int32_t* d_gaussian_ids, int64_t capacity, void* stream);
int launch_intersect_tiles(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                           int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                           void* d_workspace, int64_t workspace_bytes,
                           int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                           int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream, cudaEvent_t mark_before_sort, int64_t* d_max_pairs,
                           const int32_t* d_tile_active);
int launch_intersect_tiles_packed(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen, const int32_t* d_image_ids,
                                  const int64_t* d_total, int64_t max_pairs, int64_t n_images, int32_t width, int32_t height,
                                  void* d_workspace, int64_t workspace_bytes, int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                                  int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream, const int32_t* d_tile_active);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

struct CamDev {
    float R[9];
    float t[3];
    float fx, fy, cx, cy;
};

__device__ __forceinline__ CamDev load_cam(const float* __restrict__ viewmats, const float* __restrict__ intrins, int cid) {
    const float* m = viewmats + 16 * cid;
    CamDev c;
    c.R[0] = m[0]; c.R[1] = m[1]; c.R[2] = m[2];
    c.R[3] = m[4]; c.R[4] = m[5]; c.R[5] = m[6];
    c.R[6] = m[8]; c.R[7] = m[9]; c.R[8] = m[10];
    c.t[0] = m[3]; c.t[1] = m[7]; c.t[2] = m[11];
    c.fx = intrins[4 * cid]; c.fy = intrins[4 * cid + 1];
    c.cx = intrins[4 * cid + 2]; c.cy = intrins[4 * cid + 3];
    return c;
}

// Natural logarithm as a fixed sequence of IEEE single operations (Cephes logf), so that integers derived from it (tile
// spans, sampling order) are the same on every machine and equal the CPU statement of the same sequence.
__device__ __forceinline__ float det_logf(float xin) {
    uint32_t bits = __float_as_uint(xin);
    int e = (int)((bits >> 23) & 255u) - 127;
    float m = __uint_as_float((bits & 0x007fffffu) | 0x3f800000u);
    if (m > 1.41421356f) { m = __fmul_rn(m, 0.5f); e += 1; }
    float f = __fsub_rn(m, 1.0f);
    float z = __fmul_rn(f, f);
    float p = 7.0376836292E-2f;
    p = __fmul_rn(p, f); p = __fadd_rn(p, -1.1514610310E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 1.1676998740E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, -1.2420140846E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 1.4249322787E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, -1.6668057665E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 2.0000714765E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, -2.4999993993E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 3.3333331174E-1f);
    float fe = (float)e;
    float y = __fmul_rn(f, z); y = __fmul_rn(y, p);
    float t = __fmul_rn(-2.12194440e-4f, fe); y = __fadd_rn(y, t);
    t = __fmul_rn(0.5f, z); y = __fsub_rn(y, t);
    float r = __fadd_rn(f, y);
    t = __fmul_rn(0.693359375f, fe); r = __fadd_rn(r, t);
    return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 16-byte vector reduction into global memory (sm_90+).
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

}  // namespace ssb
