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
// Row strides of the partial maps and of their row convolution are odd (43, 33): step 4 works on two neighbouring outputs
// per thread, so a warp covers two rows with even column offsets, and an even stride would put both rows on the same banks.
constexpr int kDStride = kMid + 1, kHStride = kLossTile + 1;
constexpr int kSmemA = 3 * kMid * kDStride;           // X and Y patches (2*52*52 = 5408); later the 3 partial maps (3*42*43 = 5418)
constexpr int kSmemB = 5 * kIn * kMid;                // row-convolved moments; later 3*42*33 row-convolved partials
static_assert(kSmemA >= 2 * kIn * kIn && kSmemB >= 3 * kMid * kHStride, "shared-memory aliases must fit");
constexpr int kLossSmemBytes = (kSmemA + kSmemB) * 4;

// MAP_MODE (SsimLossMapMode, src/kernels/loss/PerPixelLoss.cuh:129-134): 0 no map; otherwise
// loss_map[pixel] += map_weight * (1 - mean over channels of v) with v = the SSIM (1), its
// contrast-structure factor D/B (2) or the structure term D / (2 sqrt(sigma1^2 sigma2^2) + C2) (3)
// (src/kernels/loss/FusedSSIM.cu:861-886,1009-1016).
template <int MAP_MODE>
__global__ void __launch_bounds__(kLossThreads) loss_l1_ssim_kernel(
    const float* __restrict__ render, const float* __restrict__ gt, int B, int H, int W,
    float w_l1, float w_ssim, float* __restrict__ v_render, float* __restrict__ losses,
    float map_weight, float* __restrict__ loss_map) {
    extern __shared__ float smem[];
    float* sX = smem;
    float* sY = smem + kIn * kIn;
    float* sM = smem + kSmemA;          // [5][kIn rows][kMid cols]
    float* sD = smem;                   // [3][kMid][kDStride]   (aliases sX/sY)
    float* sH = smem + kSmemA;          // [3][kMid rows][kHStride] (aliases sM)
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
        // 2) row convolution of the five moments: rows 0..51, centre columns 5..46.
        //    One work item = 3 neighbouring outputs of a row: 13 + 13 shared-memory reads feed
        //    15 sums (instead of 22 reads per output).
        for (int o = threadIdx.x; o < kIn * (kMid / 3); o += kLossThreads) {
            const int ly = o / (kMid / 3), lc = (o - ly * (kMid / 3)) * 3;
            const float* xr = sX + ly * kIn + lc;
            const float* yr = sY + ly * kIn + lc;
            float acc[3][5];
#pragma unroll
            for (int q = 0; q < 3; ++q)
#pragma unroll
                for (int k = 0; k < 5; ++k) acc[q][k] = 0.f;
#pragma unroll
            for (int d = 0; d < 13; ++d) {
                const float x = xr[d], y = yr[d];
                const float xx = x * x, yy = y * y, xy = x * y;
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    const int tap = d - q;
                    if (tap >= 0 && tap < 11) {
                        const float wgt = cGaussW[tap];
                        acc[q][0] += x * wgt; acc[q][1] += xx * wgt; acc[q][2] += y * wgt; acc[q][3] += yy * wgt; acc[q][4] += xy * wgt;
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 3; ++q)
#pragma unroll
                for (int k = 0; k < 5; ++k) sM[k * kIn * kMid + ly * kMid + lc + q] = acc[q][k];
        }
        __syncthreads();
        // 3) column convolution -> SSIM and its partials at the 42x42 window centres;
        //    one work item = 3 vertically neighbouring centres of a column.
        for (int o = threadIdx.x; o < (kMid / 3) * kMid; o += kLossThreads) {
            const int rg = o / kMid, c = o - rg * kMid;
            const int r0 = rg * 3;
            float m[3][5];
#pragma unroll
            for (int q = 0; q < 3; ++q)
#pragma unroll
                for (int k = 0; k < 5; ++k) m[q][k] = 0.f;
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float* col = sM + k * kIn * kMid + r0 * kMid + c;
#pragma unroll
                for (int d = 0; d < 13; ++d) {
                    const float v = col[d * kMid];
#pragma unroll
                    for (int q = 0; q < 3; ++q) {
                        const int tap = d - q;
                        if (tap >= 0 && tap < 11) m[q][k] += v * cGaussW[tap];
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const int r = r0 + q;
                const int gy = ty0 - kHalo + r, gx = tx0 - kHalo + c;
                float d0 = 0.f, d1 = 0.f, d2 = 0.f;
                if ((unsigned)gy < (unsigned)H && (unsigned)gx < (unsigned)W) {
                    const float mu1 = m[q][0], mu2 = m[q][2];
                    const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
                    const float sigma1_sq = m[q][1] - mu1_sq, sigma2_sq = m[q][3] - mu2_sq, sigma12 = m[q][4] - mu1 * mu2;
                    const float A = mu1_sq + mu2_sq + kC1;
                    const float Bv = sigma1_sq + sigma2_sq + kC2;
                    const float C_ = 2.f * mu1 * mu2 + kC1;
                    const float D_ = 2.f * sigma12 + kC2;
                    const float rAB = 1.0f / (A * Bv);
                    if (r >= kHalo && r < kHalo + kLossTile && c >= kHalo && c < kHalo + kLossTile) {
                        ssim_acc += (C_ * D_) * rAB;
                        if (MAP_MODE) {
                            float lm;
                            if (MAP_MODE == 2) lm = D_ / Bv;
                            else if (MAP_MODE == 3) lm = D_ / (2.f * sqrtf(fmaxf(sigma1_sq, 0.0f) * fmaxf(sigma2_sq, 0.0f)) + kC2);
                            else lm = (C_ * D_) * rAB;
                            // map += w * (1 - (v0 + v1 + v2) / 3) is linear in the channels' values, so each channel adds
                            // its share; the same thread meets this pixel in all three channels (no race)
                            float* slot = loss_map + (int64_t)b * P + (int64_t)gy * W + gx;
                            *slot += (ch == 0 ? map_weight : 0.f) - map_weight * (1.0f / 3.0f) * lm;
                        }
                    }
                    d0 = ((mu2 * 2.f * D_) * rAB - (mu2 * 2.f * C_) * rAB - (mu1 * 2.f * C_ * D_) * rAB / A + (mu1 * 2.f * C_ * D_) * rAB / Bv) * grad;
                    d1 = (-C_ * D_) * rAB / Bv * grad;
                    d2 = (2.f * C_) * rAB * grad;
                }
                // sD aliases the input patches, which step 2 finished reading
                const int oo = r * kDStride + c;
                sD[oo] = d0; sD[kMid * kDStride + oo] = d1; sD[2 * kMid * kDStride + oo] = d2;
            }
        }
        __syncthreads();
        // 4) row convolution of the three partial maps: rows 0..41, centre columns 5..36;
        //    one work item = 2 neighbouring outputs of a row.
        for (int o = threadIdx.x; o < kMid * (kLossTile / 2); o += kLossThreads) {
            const int r = o / (kLossTile / 2), c = (o - r * (kLossTile / 2)) * 2;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float* row = sD + k * kMid * kDStride + r * kDStride + c;
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int d = 0; d < 12; ++d) {
                    const float v = row[d];
                    if (d < 11) s0 += v * cGaussW[d];
                    if (d >= 1) s1 += v * cGaussW[d - 1];
                }
                sH[k * kMid * kHStride + r * kHStride + c] = s0;
                sH[k * kMid * kHStride + r * kHStride + c + 1] = s1;
            }
        }
        __syncthreads();
        // 5) column convolution and the gradient of this channel; one work item = 4
        //    vertically neighbouring pixels of a column (256 items = one per thread).
        for (int o = threadIdx.x; o < (kLossTile / 4) * kLossTile; o += kLossThreads) {
            const int rg = o / kLossTile, c = o - rg * kLossTile;
            const int r0 = rg * 4;
            float sacc[4][3];
#pragma unroll
            for (int q = 0; q < 4; ++q) sacc[q][0] = sacc[q][1] = sacc[q][2] = 0.f;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float* col = sH + k * kMid * kHStride + r0 * kHStride + c;
#pragma unroll
                for (int d = 0; d < 14; ++d) {
                    const float v = col[d * kHStride];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int tap = d - q;
                        if (tap >= 0 && tap < 11) sacc[q][k] += v * cGaussW[tap];
                    }
                }
            }
            const int gx = tx0 + c;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int gy = ty0 + r0 + q;
                if (gy < H && gx < W) {
                    const int64_t qi = ((int64_t)gy * W + gx) * 3 + ch;
                    const float p1 = R[qi], p2 = G[qi];
                    const float diff = p1 - p2;
                    l1_acc += fabsf(diff);
                    const float sg = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
                    V[qi] = l1_scale * sg + (sacc[q][0] + (2.f * p1) * sacc[q][1] + p2 * sacc[q][2]);
                }
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

template <int MAP_MODE>
static int launch_loss_mode(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                            float* d_v_render, float* d_losses, float map_weight, float* d_loss_map, cudaStream_t st) {
    if (int e = ensure_dynamic_smem((const void*)loss_l1_ssim_kernel<MAP_MODE>, kLossSmemBytes)) return e;
    dim3 grid((unsigned)ceil_div(W, kLossTile), (unsigned)ceil_div(H, kLossTile), (unsigned)B);
    loss_l1_ssim_kernel<MAP_MODE><<<grid, kLossThreads, kLossSmemBytes, st>>>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses,
                                                                              map_weight, d_loss_map);
    SSB_LAUNCHED("loss_l1_ssim_kernel");
    return SSB_OK;
}

int launch_loss(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                float* d_v_render, float* d_losses, cudaStream_t st) {
    return launch_loss_mode<0>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, 0.f, nullptr, st);
}

// d_losses is added to (not cleared); map_mode 0 is launch_loss
int launch_loss_map(const float* d_render, const float* d_gt, int B, int H, int W, float w_l1, float w_ssim,
                    float* d_v_render, float* d_losses, int map_mode, float map_weight, float* d_loss_map, cudaStream_t st) {
    switch (map_mode) {
        case 1: return launch_loss_mode<1>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, map_weight, d_loss_map, st);
        case 2: return launch_loss_mode<2>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, map_weight, d_loss_map, st);
        case 3: return launch_loss_mode<3>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, map_weight, d_loss_map, st);
        default: return launch_loss_mode<0>(d_render, d_gt, B, H, W, w_l1, w_ssim, d_v_render, d_losses, 0.f, nullptr, st);
    }
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

extern "C" int ssb_loss_l1_ssim_fwdbwd_map(const float* d_render, const float* d_gt, int32_t n_images, int32_t height, int32_t width,
                                           float w_l1, float w_ssim, float* d_v_render, float* d_losses,
                                           int32_t ssim_loss_map_mode, float ssim_loss_map_weight, float* d_loss_map, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_render && d_gt && d_v_render, "ssb_loss_l1_ssim_fwdbwd_map: NULL argument");
    SSB_REQUIRE(n_images >= 0 && height > 0 && width > 0, "ssb_loss_l1_ssim_fwdbwd_map: bad sizes");
    SSB_REQUIRE(ssim_loss_map_mode >= 0 && ssim_loss_map_mode <= 3, "ssb_loss_l1_ssim_fwdbwd_map: mode %d is not a SsimLossMapMode", ssim_loss_map_mode);
    SSB_REQUIRE(ssim_loss_map_mode == 0 || d_loss_map, "ssb_loss_l1_ssim_fwdbwd_map: d_loss_map is NULL");
    if (n_images == 0) return SSB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (d_losses) SSB_CUDA(cudaMemsetAsync(d_losses, 0, 3 * sizeof(float), st));
    return launch_loss_map(d_render, d_gt, n_images, height, width, w_l1, w_ssim, d_v_render, d_losses, ssim_loss_map_mode, ssim_loss_map_weight,
                           d_loss_map, st);
}
