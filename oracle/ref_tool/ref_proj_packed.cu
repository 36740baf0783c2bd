// TEST INFRASTRUCTURE.  The reference's packed projection (src/kernels/projection/ProjectionPackedFwd_kernel.cuh:16-184:
// mask kernel, inclusive scan, compacting kernel, launched in the order of launch_projection_packed_fwd_kernel,
// :292-380) and the packed mode of its projection backward kernel (src/kernels/projection/ProjectionBwd_kernel.cuh:16-130
// with camera_ids / gaussian_ids) for Vanilla3DGS<3>, PINHOLE, no distortion, on raw device buffers.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/projection/ProjectionPackedFwd_kernel.cuh"
#include "kernels/projection/ProjectionBwd_kernel.cuh"
#include <cub/cub.cuh>
#include "ref_common.cuh"
#include "ref_sync.h"

// mask [C*N] bool and scan [C*N] int64 are scratch; outputs hold `capacity` pairs.  Returns -3 when nnz > capacity.
extern "C" int ref_project_fwd_packed(
    uint32_t C, uint32_t N, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_stride,
    const float* viewmats, const float* intrins,
    bool* mask, int64_t* scan, int64_t capacity,
    int32_t* camera_ids, int32_t* gaussian_ids, float* aabb, float* depths, float* radii,
    float* xy, float* depth, float* conic, float* opac, float* rgb, int64_t* nnz_out) {
    RawWorld world(N, means, quats, scales, opacities, dc, sh);
    RawScreen screen(capacity, xy, depth, conic, opac, rgb);
    const CameraDistortionCoeffsBuffer no_dist((float*)nullptr);
    projection_packed_mask_kernel_wrapper<RefPrim, CameraModelType::PINHOLE, CameraDistortionType::None>(
        0, C, N, world, viewmats, (const float4*)intrins, no_dist, W, H, mask, sh_packed, (const float2*)sh_bounds, 15, sh_bits, sh_stride);
    size_t tmp_bytes = 0;
    cub::DeviceScan::InclusiveSum(nullptr, tmp_bytes, mask, scan, (int)(C * N));
    void* tmp = nullptr;
    cudaMalloc(&tmp, tmp_bytes);
    cub::DeviceScan::InclusiveSum(tmp, tmp_bytes, mask, scan, (int)(C * N));
    cudaFree(tmp);
    int64_t nnz = 0;
    if (C * N > 0) cudaMemcpy(&nnz, scan + ((int64_t)C * N - 1), sizeof(int64_t), cudaMemcpyDeviceToHost);
    *nnz_out = nnz;
    if (nnz > capacity) return -3;
    projection_packed_fwd_kernel_wrapper<RefPrim, CameraModelType::PINHOLE, CameraDistortionType::None>(
        0, C, N, world, viewmats, (const float4*)intrins, no_dist, W, H, scan, camera_ids, gaussian_ids, (float4*)aabb, depths, radii,
        screen, sh_packed, (const float2*)sh_bounds, 15, sh_bits, sh_stride);
    return ref_finish();
}

// Packed backward: one thread per packed pair (the kernel's N is the pair count), gradients by atomics.
extern "C" int ref_project_bwd_packed(
    uint32_t C, uint32_t N, uint32_t nnz, uint32_t W, uint32_t H,
    float* means, float* quats, float* scales, float* opacities, float* dc, float* sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_stride,
    const float* viewmats, const float* intrins, const int32_t* camera_ids, const int32_t* gaussian_ids, const float* aabb,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb,
    float* g_means, float* g_quats, float* g_scales, float* g_opacities, float* g_dc, float* g_sh) {
    RawWorld world(N, means, quats, scales, opacities, dc, sh);
    RawWorld grads(N, g_means, g_quats, g_scales, g_opacities, g_dc, g_sh);
    RawScreen v_screen((int64_t)nnz, v_xy, v_depth, v_conic, v_opac, v_rgb);
    projection_fused_bwd_kernel_wrapper<RefPrim, CameraModelType::PINHOLE, CameraDistortionType::None>(
        0, C, nnz, world, viewmats, (const float4*)intrins, CameraDistortionCoeffsBuffer((float*)nullptr), W, H,
        camera_ids, gaussian_ids, (const float4*)aabb, v_screen, grads, nullptr,
        sh_packed, (const float2*)sh_bounds, 15, sh_bits, sh_stride);
    return ref_finish();
}
