// gemm_tc.cu -- 4-bit group-64 GEMM for many activation rows ("F2": prefill chunks, large batches)
// on the 5th-generation tensor cores: tcgen05.mma (kind::f16) issued by one thread, operands in
// shared memory described by matrix descriptors, the accumulator in tensor memory (TMEM), read
// back with tcgen05.ld for the per-group scale/bias epilogue.
//
//   y[t, n] (+)= sum_g ( scale[n,g] * sum_{k in g} q[n,k] x[t,k]  +  bias[n,g] * sum_{k in g} x[t,k] )
//
// the same algebra as the GEMV family (gemv.cuh; reference SeedlessMetalForward.swift:249-258):
// the tensor core multiplies the exact 4-bit integers q (as fp16) with the fp16 activations and
// accumulates one group of 64 inputs in f32; the group's scale and bias are applied on CUDA cores.
//
// A CTA of 128 threads owns 128 weight rows (8 tiles of the fragment-major layout) and a pass of
// 32 activation rows.  Per group of 64 inputs:
//   1. every thread dequantises two fragment registers (16 nibbles of two weight rows) into the
//      A stage: K-major, no swizzle, core matrices of 8 rows x 16 bytes; 8 halves of a 16-byte
//      chunk keep the pair order (0,4,1,5,2,6,3,7) the one-logic-op dequantiser produces, and the
//      B stage stores the activations of each chunk in the same order, so no permutation is spent;
//   2. fence.proxy.async + barrier; one thread issues four MMAs (M=128, N=32, K=16 each) into
//      32 TMEM columns and commits them to an mbarrier;
//   3. all threads wait (bounded), load their row of the accumulator (tcgen05.ld 32x32b.x32:
//      thread i of the CTA <-> TMEM lane i <-> weight row i) and fold it into f32 registers.
// Nothing overlaps inside a CTA; several CTAs per SM (20 KB of shared memory, 32 TMEM columns
// each) overlap one another's phases.
#include "kernels.h"
#include "gemv.cuh"

namespace sl {

constexpr int TC_ROWS = 128;      // weight rows per CTA (UMMA M)
constexpr int TC_NT = 32;         // activation rows per pass (UMMA N)

__device__ __forceinline__ uint64_t umma_desc_kmajor(const void* smem_ptr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // shared-memory matrix descriptor: start address, leading (K-chunk) and stride (8-row group)
    // byte offsets, all without their 4 low bits; descriptor version 1; no swizzle; base offset 0
    const uint64_t addr = (uint64_t)(smem_u32(smem_ptr) >> 4) & 0x3FFFull;
    return addr | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct GemmTcArgs {
    Q4R q; int N, K, M;
    const __half* x; int ldx;
    __half* y; int ldy;
    int add_to_y;                    // y += result (residual) instead of y = result
    unsigned* err;
};

__global__ void __launch_bounds__(128) k_gemm_umma(GemmTcArgs a) {
    __shared__ __align__(128) unsigned char sA[8 * TC_ROWS * 16];      // [k-chunk][row][16 B]
    __shared__ __align__(128) unsigned char sB[8 * TC_NT * 16];        // [k-chunk][token][16 B]
    __shared__ float s_part[TC_NT][8];                                  // per token, per chunk: sum of 8 activations
    __shared__ float s_sx[TC_NT];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * TC_ROWS, t0 = blockIdx.y * TC_NT;
    const int nt = min(TC_NT, a.M - t0);
    const int G = a.K >> 6, GP = G >> 1;
    if (tid == 0) { mbar_init(&s_bar, 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"(32u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(TC_NT >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);   // f32 accumulate, f16 x f16, K-major both
    // this thread's weight row for the epilogue: row i of the CTA = tile i/16, fragment row (i%16)%8, B half (i%16)/8
    const int etile = (row0 >> 4) + (tid >> 4), er = tid & 7, eb = (tid >> 3) & 1;
    const __half* srow = reinterpret_cast<const __half*>(a.q.sr) + ((size_t)etile * GP * 8 + er) * 8 + eb * 2;   // + (g/2)*64 + (g&1)*4
    float accS[TC_NT], accB[TC_NT];
#pragma unroll
    for (int n = 0; n < TC_NT; ++n) { accS[n] = 0.f; accB[n] = 0.f; }
    bool failed = false;
    for (int g = 0; g < G; ++g) {
        // ---- 1. A stage: two fragment registers per thread (tiles warp and warp+4 of the CTA's 8) ----
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int tl = warp + 4 * h;                                   // tile inside the CTA
            const size_t T = (size_t)(row0 >> 4) + tl;
            const uint4 wv = ldg_nc_u4(a.q.wr + (T * GP + (g >> 1)) * 64 + (g & 1) * 32 + lane);
            const int r = lane >> 2, t = lane & 3;
            uint32_t d[4];
            unsigned char* pa = sA + (size_t)(2 * t) * (TC_ROWS * 16) + (size_t)(tl * 16 + r) * 16;
            dequant8(wv.x, d); *reinterpret_cast<uint4*>(pa) = make_uint4(d[0], d[1], d[2], d[3]);
            dequant8(wv.y, d); *reinterpret_cast<uint4*>(pa + TC_ROWS * 16) = make_uint4(d[0], d[1], d[2], d[3]);
            dequant8(wv.z, d); *reinterpret_cast<uint4*>(pa + 8 * 16) = make_uint4(d[0], d[1], d[2], d[3]);
            dequant8(wv.w, d); *reinterpret_cast<uint4*>(pa + TC_ROWS * 16 + 8 * 16) = make_uint4(d[0], d[1], d[2], d[3]);
        }
        // ---- B stage: 32 tokens x 8 chunks, two chunks per thread; chunk sums for the bias term ----
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int idx = tid + 128 * h, n = idx >> 3, c = idx & 7;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (n < nt) v = __ldcg(reinterpret_cast<const uint4*>(a.x + (size_t)(t0 + n) * a.ldx + g * 64 + c * 8));
            s_part[n][c] = sum8_f32(v);
            uint4 o;
            o.x = __byte_perm(v.x, v.z, 0x5410); o.y = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410); o.w = __byte_perm(v.y, v.w, 0x7632);
            *reinterpret_cast<uint4*>(sB + (size_t)c * (TC_NT * 16) + (size_t)n * 16) = o;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        // ---- 2. four MMAs of K = 16 (two 16-byte chunks each) into the 32 accumulator columns ----
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t da = umma_desc_kmajor(sA + (size_t)ks * 2 * (TC_ROWS * 16), TC_ROWS * 16, 128);
                const uint64_t db = umma_desc_kmajor(sB + (size_t)ks * 2 * (TC_NT * 16), TC_NT * 16, 128);
                umma_f16(tmem_base, da, db, idesc, ks > 0 ? 1u : 0u);
            }
            umma_commit(&s_bar);
        }
        if (tid < TC_NT) {      // the group sum of token tid, in the order the GEMV path adds its eight chunk sums
            const float* p = s_part[tid];
            s_sx[tid] = ((p[0] + p[4]) + (p[2] + p[6])) + ((p[1] + p[5]) + (p[3] + p[7]));
        }
        // ---- 3. accumulator row of this thread ----
        if (!mbar_wait_bounded(&s_bar, (uint32_t)(g & 1))) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        failed = __syncthreads_or(failed ? 1 : 0) != 0;                    // s_sx visible; everyone past the wait; one verdict for the CTA
        if (failed) break;
        uint32_t dreg[32];
        tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16), dreg);
        const __half2 sb = *reinterpret_cast<const __half2*>(srow + (size_t)(g >> 1) * 64 + (g & 1) * 4);
        const float2 f = __half22float2(sb);                               // (scale, bias) of this row and group
#pragma unroll
        for (int n = 0; n < TC_NT; ++n) {
            accS[n] = fmaf(f.x, __uint_as_float(dreg[n]), accS[n]);
            accB[n] = fmaf(f.y, s_sx[n], accB[n]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();                                                   // the stages and the accumulator may be overwritten
    }
    if (failed && a.err && tid == 0) atomicOr(a.err, 1u);
    if (!failed) {
        const int row = row0 + tid;
#pragma unroll
        for (int n = 0; n < TC_NT; ++n) {
            if (n < nt) {
                const size_t idx = (size_t)(t0 + n) * a.ldy + row;
                __half val = f2h(accS[n] + accB[n]);
                if (a.add_to_y) val = hadd_rn(a.y[idx], val);
                a.y[idx] = val;
            }
        }
    }
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(32u) : "memory");
}

int launch_gemm_tc(const Q4R& q, int N, int K, int M, const __half* x, int ldx, __half* y, int ldy, bool add_to_y, unsigned* err, cudaStream_t st) {
    if (N % TC_ROWS || K % 256) return -1;
    GemmTcArgs a{q, N, K, M, x, ldx, y, ldy, add_to_y ? 1 : 0, err};
    dim3 grid((unsigned)(N / TC_ROWS), (unsigned)((M + TC_NT - 1) / TC_NT));
    k_gemm_umma<<<grid, 128, 0, st>>>(a);
    return (int)cudaGetLastError();
}

}  // namespace sl
