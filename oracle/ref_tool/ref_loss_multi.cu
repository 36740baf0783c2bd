// TEST INFRASTRUCTURE.  The reference's multi-scale per-pixel loss driver
// (compute_multi_scale_per_pixel_losses, src/kernels/loss/PerPixelLoss.cu:941-1363), compiled from where it lies with
// the Slang-generated per-pixel code the reference ships (src/generated/per_pixel_losses.cuh), called with the colour
// modalities only: render, target, optional mask, RGB-L1 weight and SSIM weight.  The edge-aware map filters it links
// against come with the densification sources (ref_densify.cu); the modes that would call them are refused here.
#include "kernels/loss/PerPixelLoss.cu"
#include "ref_sync.h"
#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

// A host-side crash inside the reference's driver prints where it happened before the process dies.
static void segv_backtrace(int sig) {
    void* frames[64];
    int n = backtrace(frames, 64);
    const char msg[] = "ref_multi_scale_loss: fatal signal, backtrace:\n";
    (void)!write(2, msg, sizeof(msg) - 1);
    backtrace_symbols_fd(frames, n, 2);
    signal(sig, SIG_DFL);
    raise(sig);
}

static TorchTensorView view_of(const void* p, uint32_t elem, std::vector<int64_t> shape) { return TorchTensorView((uint64_t)p, elem, shape); }

// The reference reports its scalars one call late (AsyncReadout), so the driver runs twice on the same inputs; the
// gradient and the loss map of the second run are what the caller's buffers hold.
extern "C" int ref_multi_scale_loss(int num_scales, int B, int H, int W, const float* render, const float* gt, const bool* mask, int Hm, int Wm,
                                    float w_l1, float w_ssim, int loss_map_mode, float* v_render, float* loss_map_out,
                                    float* rgb_loss_out, float* ssim_out) {
    if (loss_map_mode < 0 || loss_map_mode > 4) return -1;
    signal(SIGSEGV, segv_backtrace);
    std::array<float, (int)LossWeightIndex::length> weights{};
    weights[(int)LossWeightIndex::RgbSupL1] = w_l1;
    float* v_losses = nullptr;
    cudaMalloc(&v_losses, (int)LossIndex::length * sizeof(float));
    std::vector<float> ones((int)LossIndex::length, 1.0f);      // the engine's upstream gradients: 1 for every loss,
    ones[(int)LossIndex::RgbPSNR] = 0.0f;                       // 0 for the PSNR read-out (src/engine/EngineLoss.cpp:492-502)
    cudaMemcpy(v_losses, ones.data(), ones.size() * sizeof(float), cudaMemcpyHostToDevice);
    // an absent modality: null pointer, but a four-entry shape, because the pyramid code reads the shape of every
    // modality before it tests the pointer (src/kernels/loss/PerPixelLoss.cu:1066-1073)
    TorchTensorView none((uint64_t)0, 4u, std::vector<int64_t>{0, 0, 0, 0});
    // The masked pyramid reads the shape of every rendered modality at every level (:1066-1073), so with a mask and
    // three or more levels each of them has to exist; zero images with zero weights add nothing to any term.
    float* zeros = nullptr;
    cudaMalloc(&zeros, (size_t)B * H * W * 3 * sizeof(float));
    cudaMemset(zeros, 0, (size_t)B * H * W * 3 * sizeof(float));
    TorchTensorView z1 = view_of(zeros, 4, {B, H, W, 1}), z3 = view_of(zeros, 4, {B, H, W, 3});
    std::vector<bool> needs(13, false);
    needs[0] = true;
    LossValues lv{};
    for (int rep = 0; rep < 2; ++rep) {
        PerPixelGrads grads{};
        grads.v_render_rgb = view_of(v_render, 4, {B, H, W, 3});
        lv = compute_multi_scale_per_pixel_losses(
            num_scales, view_of(render, 4, {B, H, W, 3}), view_of(gt, 4, {B, H, W, 3}), /*render_depth*/ z1, /*ref_depth*/ none, /*render_normal*/ z3,
            /*depth_normal*/ z3, /*ref_normal*/ none, /*render_Ts*/ z1, /*rgb_dist*/ z3, /*depth_dist*/ z1, /*normal_dist*/ z3, /*median_depth*/ z1,
            /*median_normal*/ z3,
            mask ? view_of(mask, 1, {B, Hm, Wm, 1}) : none, mask != nullptr, weights, w_ssim, view_of(v_losses, 4, {(int)LossIndex::length}), needs,
            (long)B, none, loss_map_out ? view_of(loss_map_out, 4, {B, H, W, 1}) : none, loss_map_mode, 0.9f, 0.0f, grads);
        cudaDeviceSynchronize();
    }
    cudaFree(v_losses);
    cudaFree(zeros);
    *rgb_loss_out = lv.rgb_loss;
    *ssim_out = lv.ssim;
    return ref_finish();
}
