// Gradient reduction and parameter distribution between the GPUs of one node, done by
// this library's own kernels over peer memory (NVLink / NVSwitch) instead of a collective
// library.
//
// The training batch is split by view: every GPU holds all parameters and, after its
// views' backward passes, a full-size gradient buffer with its partial sums
// (the reference sums the sub-batches of one GPU the same way,
// src/engine/EngineTrainStep.cpp:366-427).  Each rank owns a contiguous range of splats:
//   1. it adds its peers' partial gradients of that range to its own with ordinary loads
//      from their memory (ssb_peer_reduce_f32) -- a reduce-scatter without staging copies;
//   2. it runs Adam on the range (ssb_adam_step / ssb_adam_step_sh_quantized with a
//      sub-range), so optimiser state is touched by its owner only;
//   3. it stores the range's updated parameters into every peer's replica
//      (ssb_peer_broadcast) -- an all-gather.
// The caller separates the phases of different ranks with two stream-ordered barriers per
// iteration (before 1: every rank's backward is complete; after 3: every replica is
// complete).  No kernel waits on another GPU, so nothing here can spin.
//
// Buffers that peers access are either plain cudaMalloc allocations exported as CUDA IPC handles
// (ssb_peer_alloc/export/open) or any memory the caller has mapped on every rank; when the caller
// also has an NVSwitch multicast address for them, the sum is taken inside the switch and the
// broadcast is a multicast store (the *_mc kernels).  One process per GPU.  Peer loads bypass the L1 cache (ld.global.cv): the line a
// previous iteration left there would be stale.
#include "ssb_common.cuh"

#include <string.h>

namespace ssb {

constexpr int kPeerThreads = 256;

__device__ __forceinline__ float4 load_peer_f4(const float4* p) { return __ldcv(p); }

// own[seg] += sum over peers of peer[seg], fp32, 16 bytes per thread per step.  The number of
// ranks is a template parameter so that a thread's loads from all its peers are in flight together
// (a loop with a run-time trip count waits for each peer's data before asking the next).
template <int WORLD>
__global__ void __launch_bounds__(kPeerThreads) peer_reduce_kernel(SsbPeerTable t) {
    const int64_t stride = (int64_t)gridDim.x * kPeerThreads;
    const int64_t tid = (int64_t)blockIdx.x * kPeerThreads + threadIdx.x;
    for (int s = 0; s < t.n_segments; ++s) {
        const SsbPeerSegment sg = t.seg[s];
        float* own = (float*)((char*)t.base[sg.buffer][t.self] + sg.offset_bytes);
        const float4* peer[WORLD - 1];
#pragma unroll
        for (int k = 0; k < WORLD - 1; ++k) {
            const int p = k < t.self ? k : k + 1;                 // every rank but this one, ascending
            peer[k] = (const float4*)((const char*)t.base[sg.buffer][p] + sg.offset_bytes);
        }
        const int64_t n_vec = sg.bytes / 16;
        for (int64_t v = tid; v < n_vec; v += stride) {
            float4 x[WORLD - 1];
#pragma unroll
            for (int k = 0; k < WORLD - 1; ++k) x[k] = load_peer_f4(peer[k] + v);
            float4 acc = ((const float4*)own)[v];
#pragma unroll
            for (int k = 0; k < WORLD - 1; ++k) { acc.x += x[k].x; acc.y += x[k].y; acc.z += x[k].z; acc.w += x[k].w; }
            ((float4*)own)[v] = acc;
        }
        // the last few floats of a segment whose length is not a multiple of 16 bytes
        const int64_t tail0 = n_vec * 4, n_f = sg.bytes / 4;
        for (int64_t i = tail0 + tid; i < n_f; i += stride) {
            float acc = own[i];
#pragma unroll
            for (int k = 0; k < WORLD - 1; ++k) acc += __ldcv((const float*)peer[k] + i);
            own[i] = acc;
        }
    }
}

// peer[seg] = own[seg] for every peer.
__global__ void __launch_bounds__(kPeerThreads) peer_broadcast_kernel(SsbPeerTable t) {
    const int64_t stride = (int64_t)gridDim.x * kPeerThreads;
    const int64_t tid = (int64_t)blockIdx.x * kPeerThreads + threadIdx.x;
    for (int s = 0; s < t.n_segments; ++s) {
        const SsbPeerSegment sg = t.seg[s];
        const char* own = (const char*)t.base[sg.buffer][t.self] + sg.offset_bytes;
        const int64_t n_vec = sg.bytes / 16;
        for (int64_t v = tid; v < n_vec; v += stride) {
            const uint4 x = ((const uint4*)own)[v];
            for (int p = 0; p < t.world; ++p)
                if (p != t.self) ((uint4*)((char*)t.base[sg.buffer][p] + sg.offset_bytes))[v] = x;
        }
        for (int64_t i = n_vec * 16 + tid; i < sg.bytes; i += stride) {
            const char x = own[i];
            for (int p = 0; p < t.world; ++p)
                if (p != t.self) ((char*)t.base[sg.buffer][p] + sg.offset_bytes)[i] = x;
        }
    }
}

// The same two operations through the NVSwitch multicast address of the buffers: the switch adds
// the ranks' copies on a load (multimem.ld_reduce) and replicates a store (multimem.st).
__device__ __forceinline__ float4 multimem_sum_f4(const void* mc_addr) {
    float4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc_addr) : "memory");
    return r;
}
__device__ __forceinline__ void multimem_store_u4(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}

__global__ void __launch_bounds__(kPeerThreads) peer_reduce_mc_kernel(SsbPeerTable t) {
    const int64_t stride = (int64_t)gridDim.x * kPeerThreads;
    const int64_t tid = (int64_t)blockIdx.x * kPeerThreads + threadIdx.x;
    for (int s = 0; s < t.n_segments; ++s) {
        const SsbPeerSegment sg = t.seg[s];
        float* own = (float*)((char*)t.base[sg.buffer][t.self] + sg.offset_bytes);
        const char* mc = (const char*)t.multicast[sg.buffer] + sg.offset_bytes;
        const int64_t n_vec = sg.bytes / 16;
        int64_t v = tid;
        for (; v + 3 * stride < n_vec; v += 4 * stride) {       // four independent switch reductions in flight per thread
            const float4 r0 = multimem_sum_f4(mc + 16 * v), r1 = multimem_sum_f4(mc + 16 * (v + stride));
            const float4 r2 = multimem_sum_f4(mc + 16 * (v + 2 * stride)), r3 = multimem_sum_f4(mc + 16 * (v + 3 * stride));
            ((float4*)own)[v] = r0; ((float4*)own)[v + stride] = r1; ((float4*)own)[v + 2 * stride] = r2; ((float4*)own)[v + 3 * stride] = r3;
        }
        for (; v < n_vec; v += stride) ((float4*)own)[v] = multimem_sum_f4(mc + 16 * v);
        // the last few floats of a segment whose length is not a multiple of 16 bytes: per-peer loads
        const int64_t tail0 = n_vec * 4, n_f = sg.bytes / 4;
        for (int64_t i = tail0 + tid; i < n_f; i += stride) {
            float acc = own[i];
            for (int p = 0; p < t.world; ++p) {
                if (p == t.self) continue;
                acc += __ldcv((const float*)((const char*)t.base[sg.buffer][p] + sg.offset_bytes) + i);
            }
            own[i] = acc;
        }
    }
}

__global__ void __launch_bounds__(kPeerThreads) peer_broadcast_mc_kernel(SsbPeerTable t) {
    const int64_t stride = (int64_t)gridDim.x * kPeerThreads;
    const int64_t tid = (int64_t)blockIdx.x * kPeerThreads + threadIdx.x;
    for (int s = 0; s < t.n_segments; ++s) {
        const SsbPeerSegment sg = t.seg[s];
        const char* own = (const char*)t.base[sg.buffer][t.self] + sg.offset_bytes;
        char* mc = (char*)t.multicast[sg.buffer] + sg.offset_bytes;
        const int64_t n_vec = sg.bytes / 16;
        for (int64_t v = tid; v < n_vec; v += stride) multimem_store_u4(mc + 16 * v, ((const uint4*)own)[v]);
        for (int64_t i = n_vec * 16 + tid; i < sg.bytes; i += stride) {
            const char x = own[i];
            for (int p = 0; p < t.world; ++p)
                if (p != t.self) ((char*)t.base[sg.buffer][p] + sg.offset_bytes)[i] = x;
        }
    }
}

static bool table_has_multicast(const SsbPeerTable* t) {
    for (int s = 0; s < t->n_segments; ++s) {
        void* mc = t->multicast[t->seg[s].buffer];
        if (mc == nullptr || ((uintptr_t)mc & 15) != 0) return false;
    }
    return t->n_segments > 0;
}

static int check_table(const SsbPeerTable* t, const char* who, bool f32) {
    SSB_REQUIRE(t != nullptr, "%s: NULL table", who);
    SSB_REQUIRE(t->world >= 1 && t->world <= SSB_MAX_PEERS && t->self >= 0 && t->self < t->world, "%s: bad world/self (%d, %d)", who, t->world, t->self);
    SSB_REQUIRE(t->n_segments >= 0 && t->n_segments <= SSB_MAX_PEER_SEGMENTS, "%s: bad segment count %d", who, t->n_segments);
    for (int s = 0; s < t->n_segments; ++s) {
        const SsbPeerSegment& sg = t->seg[s];
        SSB_REQUIRE(sg.buffer >= 0 && sg.buffer < SSB_MAX_PEER_BUFFERS, "%s: segment %d names buffer %d", who, s, sg.buffer);
        SSB_REQUIRE(sg.offset_bytes >= 0 && sg.bytes >= 0, "%s: segment %d has a negative offset or length", who, s);
        if (sg.bytes == 0) continue;                 // an empty range (a rank beyond the last splat) has nothing to align
        SSB_REQUIRE((sg.offset_bytes & 15) == 0, "%s: segment %d must start on a 16-byte boundary", who, s);
        SSB_REQUIRE(!f32 || (sg.bytes & 3) == 0, "%s: segment %d is not a whole number of floats", who, s);
        for (int p = 0; p < t->world; ++p)
            SSB_REQUIRE(t->base[sg.buffer][p] != nullptr && ((uintptr_t)t->base[sg.buffer][p] & 15) == 0,
                        "%s: buffer %d of rank %d is NULL or not 16-byte aligned", who, sg.buffer, p);
    }
    return SSB_OK;
}

static unsigned peer_grid(const SsbPeerTable* t) {
    int64_t bytes = 0;
    for (int s = 0; s < t->n_segments; ++s) bytes = bytes > t->seg[s].bytes ? bytes : t->seg[s].bytes;
    const int64_t blocks = ceil_div(ceil_div(bytes, 16), kPeerThreads);
    return (unsigned)(blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks));
}

}  // namespace ssb

extern "C" {

int ssb_peer_alloc(int64_t bytes, void** d_ptr) {
    using namespace ssb;
    SSB_REQUIRE(d_ptr && bytes > 0, "ssb_peer_alloc: bad argument");
    cudaError_t e = cudaMalloc(d_ptr, (size_t)bytes);
    if (e != cudaSuccess) {
        *d_ptr = nullptr;
        set_error("ssb_peer_alloc: cudaMalloc of %lld bytes failed (%s)", (long long)bytes, cudaGetErrorString(e));
        cudaGetLastError();
        return SSB_ERR_OUT_OF_MEMORY;
    }
    SSB_CUDA(cudaMemset(*d_ptr, 0, (size_t)bytes));
    return SSB_OK;
}

int ssb_peer_free(void* d_ptr) {
    using namespace ssb;
    if (d_ptr) SSB_CUDA(cudaFree(d_ptr));
    return SSB_OK;
}

int ssb_peer_export(const void* d_ptr, unsigned char handle[SSB_PEER_HANDLE_BYTES]) {
    using namespace ssb;
    static_assert(sizeof(cudaIpcMemHandle_t) == SSB_PEER_HANDLE_BYTES, "handle size");
    SSB_REQUIRE(d_ptr && handle, "ssb_peer_export: NULL argument");
    cudaIpcMemHandle_t h;
    SSB_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(d_ptr)));
    memcpy(handle, &h, sizeof(h));
    return SSB_OK;
}

int ssb_peer_open(const unsigned char handle[SSB_PEER_HANDLE_BYTES], void** d_ptr) {
    using namespace ssb;
    SSB_REQUIRE(d_ptr && handle, "ssb_peer_open: NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    SSB_CUDA(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return SSB_OK;
}

int ssb_peer_close(void* d_ptr) {
    using namespace ssb;
    if (d_ptr) SSB_CUDA(cudaIpcCloseMemHandle(d_ptr));
    return SSB_OK;
}

int ssb_peer_reduce_f32(const SsbPeerTable* table, void* stream) {
    using namespace ssb;
    int e = check_table(table, "ssb_peer_reduce_f32", true);
    if (e) return e;
    if (table->world == 1 || table->n_segments == 0) return SSB_OK;
    if (table_has_multicast(table)) peer_reduce_mc_kernel<<<peer_grid(table), kPeerThreads, 0, (cudaStream_t)stream>>>(*table);
    else {
        const unsigned grid = peer_grid(table);
        cudaStream_t st = (cudaStream_t)stream;
        switch (table->world) {
            case 2: peer_reduce_kernel<2><<<grid, kPeerThreads, 0, st>>>(*table); break;
            case 3: peer_reduce_kernel<3><<<grid, kPeerThreads, 0, st>>>(*table); break;
            case 4: peer_reduce_kernel<4><<<grid, kPeerThreads, 0, st>>>(*table); break;
            case 5: peer_reduce_kernel<5><<<grid, kPeerThreads, 0, st>>>(*table); break;
            case 6: peer_reduce_kernel<6><<<grid, kPeerThreads, 0, st>>>(*table); break;
            case 7: peer_reduce_kernel<7><<<grid, kPeerThreads, 0, st>>>(*table); break;
            default: peer_reduce_kernel<8><<<grid, kPeerThreads, 0, st>>>(*table); break;
        }
    }
    SSB_LAUNCHED("peer_reduce_kernel");
    return SSB_OK;
}

int ssb_peer_broadcast(const SsbPeerTable* table, void* stream) {
    using namespace ssb;
    int e = check_table(table, "ssb_peer_broadcast", false);
    if (e) return e;
    if (table->world == 1 || table->n_segments == 0) return SSB_OK;
    if (table_has_multicast(table)) peer_broadcast_mc_kernel<<<peer_grid(table), kPeerThreads, 0, (cudaStream_t)stream>>>(*table);
    else peer_broadcast_kernel<<<peer_grid(table), kPeerThreads, 0, (cudaStream_t)stream>>>(*table);
    SSB_LAUNCHED("peer_broadcast_kernel");
    return SSB_OK;
}

}  // extern "C"
