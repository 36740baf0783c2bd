// Fused image loss: w_l1 * mean|render - gt| + w_ssim * (1 - SSIM) with its
// gradient with respect to the render, in one kernel.
//
// Restates the RGB-L1 term of the reference's per-pixel loss and its reverse
// (src/shaders/per_pixel_losses.slang:133-176,365-375: v = w * sign(r-g)/(3*B*P))
// and the fused SSIM forward+backward of src/kernels/loss/FusedSSIM.cu:639-1022
// (11-tap Gaussian, sigma 1.5, zero padding, C1 = 1e-4, C2 = 9e-4, gradient
// scale -w_ssim/(3*B*H*W) added on top of the L1 gradient).
//
// One CTA produces a 32x32 block of gradient pixels for all three channels.
// That needs the SSIM partial derivatives of the 42x42 window centres around
// it, hence the moments of a 52x52 input patch: the patch is loaded once per
// channel into shared memory, both separable convolutions run out of shared
// memory, and only the 32x32 gradient block is written.
#include "ssb_common.cuh"

namespace ssb {

constexpr int kLossTile = 32;
constexpr int kHalo = 5;
constexpr int kIn = kLossTile + 4 * kHalo;    // 52: input patch edge
constexpr int kMid = kLossTile + 2 * kHalo;   // 42: window-centre patch edge
constexpr int kLossThreads = 256;

__constant__ float cGaussW[11] = {
    0.001028380123898387f, 0.0075987582094967365f, 0.036000773310661316f, 0.10936068743467331f,
    0.21300552785396576f, 0.26601171493530273f, 0.21300552785396576f, 0.10936068743467331f,
    0.036000773310661316f, 0.0075987582094967365f, 0.001028380123898387f};

// shared memory layout (floats)
constexpr int kSmemA = 2 * kIn * kIn;                 // X and Y patches; later the 3 partial maps (3*42*42 = 5292 <= 5408)
constexpr int kSmemB = 5 * kIn * kMid;                // row-convolved moments; later 3*42*32 row-convolved partials
constexpr int kLossSmemBytes = (kSmemA + kSmemB) * 4;

__global__ void __launch_bounds__(kLossThreads) loss_l1_ssim_kernel(
    const float* __restrict__ render, const float* __restrict__ gt, int B, int H, int W,
    float w_l1, float w_ssim, float* __restrict__ v_render, float* __restrict__ losses) {
    extern __shared__ float smem[];
    float* sX = smem;
    float* sY = smem + kIn * kIn;
    float* sM = smem + kSmemA;          // [5][kIn rows][kMid cols]
    float* sD = smem;                   // [3][kMid][kMid]   (aliases sX/sY)
    float* sH = smem + kSmemA;          // [3][kMid rows][kLossTile cols] (aliases sM)
    __shared__ float red[2][kLossThreads / 32];

    const int b = blockIdx.z;
    const int ty0 = blockIdx.y * kLossTile, tx0 = blockIdx.x * kLossTile;
    const int64_t P = (int64_t)H * W;
    const float* R = render + (int64_t)b * P * 3;
    const float* G = gt + (int64_t)b * P * 3;
    float* V = v_render + (int64_t)b * P * 3;
    const float inv_n = 1.0f / (3.0f * (float)B * (float)W * (float)H);
    const float grad = -w_ssim * inv_n;
    const float l1_scale = w_l1 * (1.0f / 3.0f) / fmaxf((float)B * (float)P, 1.0f);
    const float kC1 = 0.01f * 0.01f, kC2 = 0.03f * 0.03f;
    float ssim_acc = 0.f, l1_acc = 0.f;

    for (int ch = 0; ch < 3; ++ch) {
        __syncthreads();
        // 1) input patch, zero padded
        for (int o = threadIdx.x; o < kIn * kIn; o += kLossThreads) {
            int ly = o / kIn, lx = o - ly * kIn;
            int gy = ty0 - 2 * kHalo + ly, gx = tx0 - 2 * kHalo + lx;
            float x = 0.f, y = 0.f;
            if ((unsigned)gy < (unsigned)H && (unsigned)gx < (unsigned)W) {
                int64_t q = ((int64_t)gy * W + gx) * 3 + ch;
                x = R[q]; y = G[q];
            }
            sX[o] = x; sY[o] = y;
        }
        __syncthreads();
        // 2) row convolution of the five moments: rows 0..51, centre columns 5..46
        for (int o = threadIdx.x; o < kIn * kMid; o += kLossThreads) {
            int ly = o / kMid, lc = o - ly * kMid;
            const float* xr = sX + ly * kIn + lc;
            const float* yr = sY + ly * kIn + lc;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, s4 = 0.f;
#pragma unroll
            for (int d = 0; d < 11; ++d) {
                float wgt = cGaussW[d], x = xr[d], y = yr[d];
                s0 += x * wgt; s1 += x * x * wgt; s2 += y * wgt; s3 += y * y * wgt; s4 += x * y * wgt;
            }
            sM[0 * kIn * kMid + o] = s0; sM[1 * kIn * kMid + o] = s1; sM[2 * kIn * kMid + o] = s2;
            sM[3 * kIn * kMid + o] = s3; sM[4 * kIn * kMid + o] = s4;
        }
        __syncthreads();
        // 3) column convolution -> SSIM and its partials at the 42x42 window centres
        for (int o = threadIdx.x; o < kMid * kMid; o += kLossThreads) {
            int r = o / kMid, c = o - r * kMid;
            float m[5];
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float* col = sM + k * kIn * kMid + r * kMid + c;
                float s = 0.f;
#pragma unroll
                for (int d = 0; d < 11; ++d) s += col[d * kMid] * cGaussW[d];
                m[k] = s;
            }
            int gy = ty0 - kHalo + r, gx = tx0 - kHalo + c;
            float d0 = 0.f, d1 = 0.f, d2 = 0.f;
            if ((unsigned)gy < (unsigned)H && (unsigned)gx < (unsigned)W) {
                float mu1 = m[0], mu2 = m[2];
                float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
                float sigma1_sq = m[1] - mu1_sq, sigma2_sq = m[3] - mu2_sq, sigma12 = m[4] - mu1 * mu2;
                float A = mu1_sq + mu2_sq + kC1;
                float Bv = sigma1_sq + sigma2_sq + kC2;
                float C_ = 2.f * mu1 * mu2 + kC1;
                float D_ = 2.f * sigma12 + kC2;
                float rAB = 1.0f / (A * Bv);
                if (r >= kHalo && r < kHalo + kLossTile && c >= kHalo && c < kHalo + kLossTile) ssim_acc += (C_ * D_) * rAB;
                d0 = ((mu2 * 2.f * D_) * rAB - (mu2 * 2.f * C_) * rAB - (mu1 * 2.f * C_ * D_) * rAB / A + (mu1 * 2.f * C_ * D_) * rAB / Bv) * grad;
                d1 = (-C_ * D_) * rAB / Bv * grad;
                d2 = (2.f * C_) * rAB * grad;
            }
            // sD aliases the input patches, which step 2 finished reading
            sD[o] = d0; sD[kMid * kMid + o] = d1; sD[2 * kMid * kMid + o] = d2;
        }
        __syncthreads();
        // 4) row convolution of the three partial maps: rows 0..41, centre columns 5..36
        for (int o = threadIdx.x; o < kMid * kLossTile; o += kLossThreads) {
            int r = o / kLossTile, c = o - r * kLossTile;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float* row = sD + k * kMid * kMid + r * kMid + c;
                float s = 0.f;
#pragma unroll
                for (int d = 0; d < 11; ++d) s += row[d] * cGaussW[d];
                sH[k * kMid * kLossTile + o] = s;
            }
        }
        __syncthreads();
        // 5) column convolution and the gradient of this channel
        for (int o = threadIdx.x; o < kLossTile * kLossTile; o += kLossThreads) {
            int r = o / kLossTile, c = o - r * kLossTile;
            int gy = ty0 + r, gx = tx0 + c;
            if (gy < H && gx < W) {
                float s[3];
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    const float* col = sH + k * kMid * kLossTile + r * kLossTile + c;
                    float a = 0.f;
#pragma unroll
                    for (int d = 0; d < 11; ++d) a += col[d * kLossTile] * cGaussW[d];
                    s[k] = a;
                }
                int64_t q = ((int64_t)gy * W + gx) * 3 + ch;
                float p1 = R[q], p2 = G[q];
                float diff = p1 - p2;
                l1_acc += fabsf(diff);
                float sg = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
                V[q] = l1_scale * sg + (s[0] + (2.f * p1) * s[1] + p2 * s[2]);
            }
        }
    }
    // block reduction of the two scalars
    ssim_acc = warp_sum(ssim_acc);
    l1_acc = warp_sum(l1_acc);
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = ssim_acc; red[1][threadIdx.x >> 5] = l1_acc; }
    __syncthreads();
    if (threadIdx.x == 0 && losses) {
        float s = 0.f, l = 0.f;
        for (int k = 0; k < kLossThreads / 32; ++k) { s += red[0][k]; l += red[1][k]; }
        float l1_mean = l * inv_n, ssim_mean = s * inv_n;
        atomicAdd(&losses[0], l1_mean);
        atomicAdd(&losses[1], ssim_mean);
        float tot = w_l1 * l1_mean - w_ssim * ssim_mean;
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) tot += w_ssim;
        atomicAdd(&losses[2], tot);
    }
}

int launch_loss(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                float* d_v_render, float* d_losses, cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        SSB_CUDA(cudaFuncSetAttribute(loss_l1_ssim_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLossSmemBytes));
        attr_set = true;
    }
    dim3 grid((unsigned)ceil_div(W, kLossTile), (unsigned)ceil_div(H, kLossTile), (unsigned)B);
    loss_l1_ssim_kernel<<<grid, kLossThreads, kLossSmemBytes, st>>>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses);
    SSB_LAUNCHED("loss_l1_ssim_kernel");
    return SSB_OK;
}

}  // namespace ssb

extern "C" int ssb_loss_l1_ssim_fwdbwd(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                                       float w_l1, float w_ssim, float* d_v_render, float* d_losses, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_render && d_gt && d_v_render, "ssb_loss_l1_ssim_fwdbwd: NULL argument");
    SSB_REQUIRE(n_images >= 0 && height > 0 && width > 0, "ssb_loss_l1_ssim_fwdbwd: bad sizes");
    if (n_images == 0) return SSB_OK;
    if (d_losses) SSB_CUDA(cudaMemsetAsync(d_losses, 0, 3 * sizeof(float), (cudaStream_t)stream));
    return launch_loss(d_render, d_gt, n_images, height, width, w_l1, w_ssim, d_v_render, d_losses, (cudaStream_t)stream);
}
