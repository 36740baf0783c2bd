// TEST INFRASTRUCTURE.  The reference's fused SSIM forward+backward kernel
// (src/kernels/loss/FusedSSIM.cu:639-1022), launched as fused_ssim_inplace does
// (:1163-1176) with no mask and no loss map: adds the SSIM gradient into dL_dimg1
// and the mean SSIM into *ssim_out.
#include "kernels/loss/FusedSSIM.cu"
#include "ref_sync.h"

extern "C" int ref_ssim_inplace(int B, int H, int W, const float* img1, const float* img2, float dL_dmap, float* dL_dimg1, float* ssim_out) {
    cudaMemset(ssim_out, 0, sizeof(float));
    memory_efficient_ssim_backward_kernel<true><<<_LAUNCH_ARGS_3D(W, H, B, BLOCK_X_ME, BLOCK_Y_ME, 1)>>>(
        B, H, W, (const float3*)img1, (const float3*)img2, nullptr, 0, 0, 0, nullptr, dL_dmap, (float3*)dL_dimg1, ssim_out, 0.0f, nullptr, 0);
    return ref_finish();
}

// The same launch with the densification loss map (fused_ssim_inplace_async's ssim_loss_map arguments, :1211-1234):
// loss_map += weight * (1 - SSIM variant), mode = SsimLossMapMode 1..3.
extern "C" int ref_ssim_inplace_map(int B, int H, int W, const float* img1, const float* img2, float dL_dmap, float* dL_dimg1, float* ssim_out,
                                    float map_weight, float* loss_map, int mode) {
    cudaMemset(ssim_out, 0, sizeof(float));
    memory_efficient_ssim_backward_kernel<true><<<_LAUNCH_ARGS_3D(W, H, B, BLOCK_X_ME, BLOCK_Y_ME, 1)>>>(
        B, H, W, (const float3*)img1, (const float3*)img2, nullptr, 0, 0, 0, nullptr, dL_dmap, (float3*)dL_dimg1, ssim_out, map_weight, loss_map, mode);
    return ref_finish();
}

// The masked launch, as fused_ssim_inplace does it (:1140-1176): the window coverage of the mask from
// _ssim_mask_coverage (:181-195), then the kernel with the mask, its own dimensions and the coverage.  mask is
// [Bm][Hm][Wm] bool (one byte each).  map_mode 0 leaves loss_map alone.
extern "C" int ref_ssim_inplace_masked(int B, int H, int W, const float* img1, const float* img2, const bool* mask, int Bm, int Hm, int Wm,
                                       float dL_dmap, float* dL_dimg1, float* ssim_out, float map_weight, float* loss_map, int mode) {
    cudaMemset(ssim_out, 0, sizeof(float));
    const float* mask_w = _ssim_mask_coverage(B, H, W, mask, Bm, Hm, Wm);
    memory_efficient_ssim_backward_kernel<true><<<_LAUNCH_ARGS_3D(W, H, B, BLOCK_X_ME, BLOCK_Y_ME, 1)>>>(
        B, H, W, (const float3*)img1, (const float3*)img2, mask, Bm, Hm, Wm, mask_w, dL_dmap, (float3*)dL_dimg1, ssim_out, map_weight, loss_map, mode);
    return ref_finish();
}
