// common.cuh -- shared device helpers for the Seedless B200 kernels (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sl {

// fixed by the model family (swift/Sources/QwispCore/QwispModel.swift:83-120)
constexpr int GDN_DK = 128;      // gated-delta key head dim
constexpr int GDN_DV = 128;      // gated-delta value head dim
constexpr int CONV_K = 4;        // causal depthwise conv taps
constexpr int ATT_D = 256;       // attention head dim
constexpr int ROPE_D = 64;       // rotated dims (NeoX pairs d, d+32)
constexpr int QGROUP = 64;       // quantisation group

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}
// sum over aligned groups of 16 lanes
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }
__device__ __forceinline__ __half f2h(float f) { return __float2half_rn(f); }

// correctly rounded fp16 arithmetic done through one f32 operation (f32 carries >= 2*11+2 bits)
__device__ __forceinline__ __half hadd_rn(__half a, __half b) { return f2h(__fadd_rn(h2f(a), h2f(b))); }
__device__ __forceinline__ __half hsub_rn(__half a, __half b) { return f2h(__fsub_rn(h2f(a), h2f(b))); }
__device__ __forceinline__ __half hmul_rn(__half a, __half b) { return f2h(__fmul_rn(h2f(a), h2f(b))); }
__device__ __forceinline__ __half hdiv_rn(__half a, __half b) { return f2h(__fdiv_rn(h2f(a), h2f(b))); }

// "stable sigmoid" in fp16 arithmetic: y = 1/(1+exp(|x|)); x<0 ? y : 1-y
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:986-988)
__device__ __forceinline__ __half sigmoid_h(__half x) {
    const __half one = f2h(1.0f);
    __half ex = f2h(expf(fabsf(h2f(x))));
    __half y = hdiv_rn(one, hadd_rn(one, ex));
    return (h2f(x) < 0.0f) ? y : hsub_rn(one, y);
}
// same in f32 (SeedlessMetalForward.swift:1599-1602)
__device__ __forceinline__ float sigmoid_f(float x) {
    float y = __fdiv_rn(1.0f, 1.0f + expf(fabsf(x)));
    return (x < 0.0f) ? y : (1.0f - y);
}
// SwiGLU in fp16: (g*sigmoid(g))*u (SeedlessMetalForward.swift:982-990)
__device__ __forceinline__ __half swiglu_h(__half g, __half u) { return hmul_rn(hmul_rn(g, sigmoid_h(g)), u); }

// Programmatic dependent launch: wait for the kernels this one depends on / let dependents start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// L2 prefetch of [p, p+bytes): bytes a multiple of 16, p 16-byte aligned
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// ---- bulk asynchronous copies global -> shared, completion counted on an mbarrier (no multicast) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
// dst and src 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* b) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (seconds) so a copy that never lands cannot hang the GPU;
// the caller records the failure and carries on with whatever is in shared memory.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* b, uint32_t parity, int limit = 1 << 22) {
    for (int i = 0; i < limit; ++i) if (mbar_try_wait(b, parity)) return true;
    return false;
}

__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_nc_u2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// ---- cross-GPU flags of the expert-parallel exchange (system scope: the other side is a peer GPU) ----
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// sequence number of (step counter, MoE layer of the step, phase 0 = dispatch / 1 = combine): monotonic, never 0
__device__ __forceinline__ unsigned ep_seq(const unsigned* ctr, int layer, int phase) { return (*ctr) * 256u + (unsigned)layer * 2u + (unsigned)phase + 1u; }

// per-stream device-resident bookkeeping, indexed by stream slot
struct StreamTable {
    int* kv_len;            // [max_streams] positions already in the cache
    int* parity;            // [max_streams] which GDN ping-pong side is current
    int* page_table;        // [max_streams][max_pages]
    int max_pages;
    float* gdn_state;       // [max_streams][2][n_gdn][Hv][128][128]
    __half* conv_hist;      // [max_streams][2][n_gdn][3][convDim]
    size_t state_stride_layer, state_stride_side, state_stride_stream;   // in floats
    size_t hist_stride_layer, hist_stride_side, hist_stride_stream;      // in halfs
};

// rows of one call: segment = contiguous rows of one stream, in sequence order
struct SegDesc { int slot; int row0; int nrows; int pad; };

}  // namespace sl
