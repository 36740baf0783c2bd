// TEST INFRASTRUCTURE.  Runs the reference's OWN tile-intersection device code
// (src/kernels/tile/IntersectTile.cu, included from where it lies in the
// reference tree) on raw device buffers, following the launch sequence of
// do_intersect_tile_generic (src/kernels/tile/IntersectTile.cu:372-509):
// count kernel -> cub inclusive scan -> key kernel -> cub radix sort -> offset kernel.
#include "kernels/tile/IntersectTile.cu"
#include "ref_sync.h"

// tile_active: the live-tile map [I][tile_h][tile_w] or NULL (every tile live), as do_intersect_tile_generic takes it.
static int intersect_tile_sequence(
    uint32_t I, uint32_t N, uint32_t W, uint32_t H,
    const float* aabb, const float* depths, const float* xy, const float* conic, const float* opac, const int32_t* tile_active,
    int64_t* tiles_per_splat, int64_t* cum_tiles, int64_t capacity,
    int64_t* ids_a, int64_t* ids_b, int32_t* flat_a, int32_t* flat_b, int32_t* offsets,
    int64_t* n_isects_out, int32_t* selector_out) {
    uint32_t tile_width = _CEIL_DIV(W, TILE_SIZE_IX), tile_height = _CEIL_DIV(H, TILE_SIZE_IY);
    uint32_t n_tiles = tile_width * tile_height * I;
    uint32_t total = I * N;
    intersect_tile_kernel<true, true><<<_CEIL_DIV(total, 256), 256>>>(
        I, N, nullptr, nullptr, (const float4*)aabb, depths, (const float2*)xy, (const float3*)conic, opac, nullptr,
        tile_width, tile_height, tile_active, tiles_per_splat, nullptr, nullptr);
    size_t tmp_bytes = 0;
    cub::DeviceScan::InclusiveSum(nullptr, tmp_bytes, tiles_per_splat, cum_tiles, (int)total);
    void* tmp = nullptr;
    cudaMalloc(&tmp, tmp_bytes);
    cub::DeviceScan::InclusiveSum(tmp, tmp_bytes, tiles_per_splat, cum_tiles, (int)total);
    cudaFree(tmp);
    int64_t n_isects = 0;
    cudaMemcpy(&n_isects, cum_tiles + (total - 1), sizeof(int64_t), cudaMemcpyDeviceToHost);
    *n_isects_out = n_isects;
    *selector_out = 0;
    if (n_isects > capacity) return -3;
    if (n_isects == 0) { cudaMemset(offsets, 0, sizeof(int32_t) * n_tiles); return ref_finish(); }
    intersect_tile_kernel<false, true><<<_CEIL_DIV(total, 256), 256>>>(
        I, N, nullptr, nullptr, (const float4*)aabb, depths, (const float2*)xy, (const float3*)conic, opac, cum_tiles,
        tile_width, tile_height, tile_active, nullptr, ids_a, flat_a);
    cub::DoubleBuffer<int64_t> d_keys(ids_a, ids_b);
    cub::DoubleBuffer<int32_t> d_values(flat_a, flat_b);
    int tile_n_bits = 0;
    while ((1U << tile_n_bits) <= n_tiles) ++tile_n_bits;
    tmp_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, d_keys, d_values, n_isects, 0, 32 + tile_n_bits);
    cudaMalloc(&tmp, tmp_bytes);
    cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, d_keys, d_values, n_isects, 0, 32 + tile_n_bits);
    cudaFree(tmp);
    *selector_out = d_keys.selector;
    intersect_offset_kernel<<<_CEIL_DIV((uint32_t)n_isects, 256), 256>>>(
        (uint32_t)n_isects, d_keys.selector ? ids_b : ids_a, I, tile_width, tile_height, offsets);
    return ref_finish();
}


extern "C" int ref_intersect_tile(
    uint32_t I, uint32_t N, uint32_t W, uint32_t H,
    const float* aabb, const float* depths, const float* xy, const float* conic, const float* opac,
    int64_t* tiles_per_splat, int64_t* cum_tiles, int64_t capacity,
    int64_t* ids_a, int64_t* ids_b, int32_t* flat_a, int32_t* flat_b, int32_t* offsets,
    int64_t* n_isects_out, int32_t* selector_out) {
    return intersect_tile_sequence(I, N, W, H, aabb, depths, xy, conic, opac, nullptr, tiles_per_splat, cum_tiles, capacity, ids_a, ids_b, flat_a,
                                   flat_b, offsets, n_isects_out, selector_out);
}

// The live-tile map of a mask (compute_tile_active, :354-367) and the intersection that skips the tiles it marks 0.
extern "C" int ref_tile_active(const bool* mask, int I, int H_mask, int W_mask, int W, int H, int32_t* tile_active) {
    const uint32_t tile_width = _CEIL_DIV((uint32_t)W, TILE_SIZE_IX), tile_height = _CEIL_DIV((uint32_t)H, TILE_SIZE_IY);
    const uint32_t n_tiles = (uint32_t)I * tile_width * tile_height;
    tile_active_kernel<<<_LAUNCH_ARGS_1D(n_tiles, 256)>>>(mask, I, H_mask, W_mask, W, H, tile_width, tile_height, tile_active);
    return ref_finish();
}

extern "C" int ref_intersect_tile_live(
    uint32_t I, uint32_t N, uint32_t W, uint32_t H,
    const float* aabb, const float* depths, const float* xy, const float* conic, const float* opac, const int32_t* tile_active,
    int64_t* tiles_per_splat, int64_t* cum_tiles, int64_t capacity,
    int64_t* ids_a, int64_t* ids_b, int32_t* flat_a, int32_t* flat_b, int32_t* offsets,
    int64_t* n_isects_out, int32_t* selector_out) {
    return intersect_tile_sequence(I, N, W, H, aabb, depths, xy, conic, opac, tile_active, tiles_per_splat, cum_tiles, capacity, ids_a, ids_b, flat_a,
                                   flat_b, offsets, n_isects_out, selector_out);
}


// The same sequence for a timing harness: the cub temp storage is the caller's (the reference keeps one
// grow-only DeviceScratch, src/core/Common.cuh:228-234, so a steady-state step allocates nothing), while the
// host read of the pair count stays, as in do_intersect_tile_generic (src/kernels/tile/IntersectTile.cu:432-436).
extern "C" int ref_intersect_tile_prealloc(
    uint32_t I, uint32_t N, uint32_t W, uint32_t H,
    const float* aabb, const float* depths, const float* xy, const float* conic, const float* opac,
    int64_t* tiles_per_splat, int64_t* cum_tiles, int64_t capacity,
    int64_t* ids_a, int64_t* ids_b, int32_t* flat_a, int32_t* flat_b, int32_t* offsets,
    void* tmp, int64_t tmp_capacity, int64_t* n_isects_out, int32_t* selector_out) {
    uint32_t tile_width = _CEIL_DIV(W, TILE_SIZE_IX), tile_height = _CEIL_DIV(H, TILE_SIZE_IY);
    uint32_t n_tiles = tile_width * tile_height * I;
    uint32_t total = I * N;
    intersect_tile_kernel<true, true><<<_CEIL_DIV(total, 256), 256>>>(
        I, N, nullptr, nullptr, (const float4*)aabb, depths, (const float2*)xy, (const float3*)conic, opac, nullptr,
        tile_width, tile_height, nullptr, tiles_per_splat, nullptr, nullptr);
    size_t tmp_bytes = 0;
    cub::DeviceScan::InclusiveSum(nullptr, tmp_bytes, tiles_per_splat, cum_tiles, (int)total);
    if ((int64_t)tmp_bytes > tmp_capacity) return -4;
    cub::DeviceScan::InclusiveSum(tmp, tmp_bytes, tiles_per_splat, cum_tiles, (int)total);
    int64_t n_isects = 0;
    cudaMemcpy(&n_isects, cum_tiles + (total - 1), sizeof(int64_t), cudaMemcpyDeviceToHost);
    *n_isects_out = n_isects;
    *selector_out = 0;
    if (n_isects > capacity) return -3;
    if (n_isects == 0) { cudaMemset(offsets, 0, sizeof(int32_t) * n_tiles); return ref_finish(); }
    intersect_tile_kernel<false, true><<<_CEIL_DIV(total, 256), 256>>>(
        I, N, nullptr, nullptr, (const float4*)aabb, depths, (const float2*)xy, (const float3*)conic, opac, cum_tiles,
        tile_width, tile_height, nullptr, nullptr, ids_a, flat_a);
    cub::DoubleBuffer<int64_t> d_keys(ids_a, ids_b);
    cub::DoubleBuffer<int32_t> d_values(flat_a, flat_b);
    int tile_n_bits = 0;
    while ((1U << tile_n_bits) <= n_tiles) ++tile_n_bits;
    tmp_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, d_keys, d_values, n_isects, 0, 32 + tile_n_bits);
    if ((int64_t)tmp_bytes > tmp_capacity) return -4;
    cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, d_keys, d_values, n_isects, 0, 32 + tile_n_bits);
    *selector_out = d_keys.selector;
    intersect_offset_kernel<<<_CEIL_DIV((uint32_t)n_isects, 256), 256>>>(
        (uint32_t)n_isects, d_keys.selector ? ids_b : ids_a, I, tile_width, tile_height, offsets);
    return ref_finish();
}
