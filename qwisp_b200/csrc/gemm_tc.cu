// gemm_tc.cu -- 4-bit group-64 GEMM for many activation rows ("F2": prompt chunks in prefill mode) on the 5th-generation
// tensor cores: tcgen05.mma (kind::f16) issued by one thread, operands in shared memory described by matrix
// descriptors, the accumulator in tensor memory (TMEM), read back once with tcgen05.ld.
//
//   y[t, n] (+)= sum_k x[t, k] * fp16(scale[n, k/64] * q[n, k] + bias[n, k/64])
//
// Prefill-mode numerics: every weight is dequantised to fp16 with one rounding (the dequantised-weight GEMM of the
// reference's batched / prefill path, swift/Sources/QwispCore/SeedlessMetalForward.swift:160-185), so the whole K
// range accumulates in ONE f32 accumulator in TMEM and the epilogue runs once.  Like the reference's hybrid prefill
// this is not bit-identical to the GEMV family, but every token column is independent of the others and K is walked in
// a fixed order, so results do not depend on how many rows share a call or on how a prompt is cut into calls.
//
// A CTA of 256 threads owns 128 weight rows (8 tiles of the fragment-major layout, one per warp) and NT activation rows.
// Four shared-memory stages rotate over the K groups of 64 inputs; per group
//   B  the NT x 64 activations go global -> shared memory by cp.async (16-byte pieces, no registers), issued TWO groups
//      ahead into the stage whose MMAs of four groups ago have completed;
//   A  each warp dequantises its tile's fragment register (16 nibbles of two weight rows; scale and bias applied with one
//      fp16x2 multiply-add per pair; halves put back in natural order) into the stage -- the register was loaded two
//      groups ahead;
//   two groups share one cp.async.wait_group + fence.proxy.async + barrier, after which one thread issues eight MMAs
//   (M=128, N=NT, K=16) that accumulate into the NT TMEM columns and commits them to a stage mbarrier.
// Operand tiles are K-major with the 128-byte swizzle (an unswizzled layout ran the same MMAs several times slower).
#include "kernels.h"
#include "gemv.cuh"

namespace sl {

constexpr int TC_ROWS = 128;      // weight rows per CTA (UMMA M)

// Operand tiles in shared memory: K-major, 128-byte swizzle.  A row holds the 64 halves of one K group (128 bytes); 8 rows
// form a 1024-byte atom inside which the 16-byte chunk index is XORed with the row index (conflict-free for the threads
// that fill it and for the tensor core that reads it); atoms of further rows follow at 1024-byte steps.  Tiles start on
// 1024-byte boundaries.
__device__ __forceinline__ unsigned char* tc_at(unsigned char* tile, int row, int chunk) {
    return tile + ((size_t)(row >> 3) << 10) + ((row & 7) << 7) + (((chunk ^ row) & 7) << 4);
}
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_ptr) {
    // shared-memory matrix descriptor: start address; leading byte offset 1 (unused by swizzled K-major layouts); stride
    // byte offset 1024 (between 8-row atoms); all without their 4 low bits; descriptor version 1; layout type 2 = 128-byte swizzle
    const uint64_t addr = (uint64_t)(smem_u32(smem_ptr) >> 4) & 0x3FFFull;
    return addr | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
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

// Short wait on a stage barrier: non-blocking polls (the MMAs it waits for take a few hundred nanoseconds; a blocking
// try_wait may park the warp for longer than that), bounded like every wait.
__device__ __forceinline__ bool tc_wait(uint64_t* b, uint32_t parity) {
    for (int i = 0; i < (1 << 24); ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// ---- pieces of a K group shared by the dense and the grouped-expert kernels ----
constexpr int TC_STAGES = 4;
constexpr int TC_THREADS = 256;
// fragment register of one 16-row tile (wv: nibbles of rows A_r / B_r, sv: their scales and biases for the pair of groups)
// -> fp16 weights, natural order, in the A stage
__device__ __forceinline__ void tc_dequant_A(unsigned char* sA, int tl, int r, int t, int g, uint4 wv, uint4 sv, bool valid) {
    uint4 o[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (valid) {
        const uint32_t sa = (g & 1) ? sv.z : sv.x, sb = (g & 1) ? sv.w : sv.y;         // (scale, bias) of rows A_r and B_r
        const __half2 hA = *reinterpret_cast<const __half2*>(&sa), hB = *reinterpret_cast<const __half2*>(&sb);
        const __half2 sA2 = __half2half2(__low2half(hA)), bA2 = __half2half2(__high2half(hA));
        const __half2 sB2 = __half2half2(__low2half(hB)), bB2 = __half2half2(__high2half(hB));
        const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            uint32_t d[4], w[4];
            dequant8(words[wi], d);                                    // (q0,q4) (q1,q5) (q2,q6) (q3,q7)
            const __half2 sc = (wi < 2) ? sA2 : sB2, bi = (wi < 2) ? bA2 : bB2;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 wq = __hfma2(*reinterpret_cast<const __half2*>(&d[j]), sc, bi);
                w[j] = *reinterpret_cast<const uint32_t*>(&wq);
            }
            o[wi].x = __byte_perm(w[0], w[1], 0x5410);                 // (w0, w1)
            o[wi].y = __byte_perm(w[2], w[3], 0x5410);                 // (w2, w3)
            o[wi].z = __byte_perm(w[0], w[1], 0x7632);                 // (w4, w5)
            o[wi].w = __byte_perm(w[2], w[3], 0x7632);                 // (w6, w7)
        }
    }
    const int rowA = tl * 16 + r;                                     // row A_r of the tile; B_r is 8 rows further (the next atom)
    *reinterpret_cast<uint4*>(tc_at(sA, rowA, 2 * t)) = o[0];
    *reinterpret_cast<uint4*>(tc_at(sA, rowA, 2 * t + 1)) = o[1];
    *reinterpret_cast<uint4*>(tc_at(sA, rowA + 8, 2 * t)) = o[2];
    *reinterpret_cast<uint4*>(tc_at(sA, rowA + 8, 2 * t + 1)) = o[3];
}
// piece idx of the B stage: token = 8 * (idx / 64) + idx % 8, chunk = (idx / 8) % 8 -- the 8 lanes of a quarter warp write
// into the 8 rows of one atom (distinct swizzled chunks) and read 4 x 64 contiguous bytes per token row
__device__ __forceinline__ void tc_piece(int idx, int& n, int& c) { n = ((idx >> 6) << 3) + (idx & 7); c = (idx >> 3) & 7; }
__device__ __forceinline__ void tc_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// The K loop of one output tile.  load_a(g, wv, sv): this warp's fragment register of group g; b_src(n): global address
// of token row n's first input, or nullptr (the row stays zero).  cb: commits made on the barriers of stages 1 and 3 by
// earlier tiles of this CTA (a tile adds G/4 to each; G is a multiple of 4); advanced here.  Returns false if a wait ran out.
template <int NT, class LoadA, class BSrc>
__device__ __forceinline__ bool tc_mainloop(unsigned char* smem, uint64_t* s_bar, int& cb, uint32_t tmem_base, int G, bool tvalid,
                                            LoadA load_a, BSrc b_src) {
    constexpr int A_BYTES = TC_ROWS * 128, B_BYTES = NT * 128, STAGE = A_BYTES + B_BYTES, NB = NT * 8 / TC_THREADS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, t = lane & 3;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);   // f32 accumulate, f16 x f16, K-major both
    bool ok = true;
    // this thread's pieces of the B tile: source row pointer (or null) and offset inside a stage
    const __half* bsrc[NB]; uint32_t boff[NB];
#pragma unroll
    for (int h = 0; h < NB; ++h) {
        int n, c; tc_piece(tid + TC_THREADS * h, n, c);
        const __half* p = b_src(n);
        bsrc[h] = p ? p + c * 8 : nullptr;
        boff[h] = (uint32_t)(tc_at(smem + A_BYTES, n, c) - smem);
        if (!p) {
#pragma unroll
            for (int s = 0; s < TC_STAGES; ++s) *reinterpret_cast<uint4*>(smem + (size_t)s * STAGE + boff[h]) = make_uint4(0, 0, 0, 0);
        }
    }
    auto issue_b = [&](int g) {
        unsigned char* st = smem + (size_t)(g % TC_STAGES) * STAGE;
#pragma unroll
        for (int h = 0; h < NB; ++h) if (bsrc[h]) tc_cp16(st + boff[h], bsrc[h] + g * 64);
    };
    uint4 wv0, sv0, wv1, sv1;                                              // fragment registers of groups g and g + 1
    if (tvalid) { load_a(0, wv0, sv0); load_a(1, wv1, sv1); }
    issue_b(0); issue_b(1);
    tc_cp_commit();
    // Two groups per barrier: B of the NEXT pair is requested first (its stages were last read by the MMAs of the pair
    // before this one), then both A tiles of this pair are dequantised, then one wait + fence + barrier and eight MMAs.
    for (int g = 0; g < G; g += 2) {                                       // G is a multiple of 4 (K is a multiple of 256)
        const int s0 = g % TC_STAGES, s1 = s0 + 1;
        unsigned char* sA0 = smem + (size_t)s0 * STAGE;
        unsigned char* sA1 = smem + (size_t)s1 * STAGE;
        if (g + 2 < G) {
            // stages (g + 2) % 4 and (g + 3) % 4 were used by groups g - 2 and g - 1: their commit is the one on stage (g + 3) % 4
            const int s3 = (g + 3) % TC_STAGES;
            if (g >= 2 && !tc_wait(&s_bar[s3], (uint32_t)((cb + (g + 3) / TC_STAGES - 1) & 1))) ok = false;
            issue_b(g + 2); issue_b(g + 3);
        }
        tc_cp_commit();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tc_dequant_A(sA0, warp, r, t, g, wv0, sv0, tvalid);
        tc_dequant_A(sA1, warp, r, t, g + 1, wv1, sv1, tvalid);
        if (tvalid && g + 2 < G) { load_a(g + 2, wv0, sv0); load_a(g + 3, wv1, sv1); }
        asm volatile("cp.async.wait_group 1;" ::: "memory");               // B of this pair has landed (the next pair may be in flight)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                unsigned char* sA = (ks < 4) ? sA0 : sA1;
                const uint64_t da = umma_desc_sw128(sA + (ks & 3) * 32), db = umma_desc_sw128(sA + A_BYTES + (ks & 3) * 32);
                umma_f16(tmem_base, da, db, idesc, (g > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(&s_bar[s1]);                                       // one commit per pair, on the odd stage's barrier
        }
    }
    // the last commit covers every MMA issued before it
    cb += G / TC_STAGES;                                                   // commits so far on the barriers of stages 1 and 3
    if (!tc_wait(&s_bar[(G - 1) % TC_STAGES], (uint32_t)((cb - 1) & 1))) ok = false;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    return ok;
}

struct GemmTcArgs {
    Q4R q; int N, K, M;
    const __half* x; int ldx;
    __half* y; int ldy;
    int add_to_y;                    // y += result (residual) instead of y = result
    unsigned* err;
};

template <int NT>
__global__ void __launch_bounds__(TC_THREADS, 1) k_gemm_umma(GemmTcArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];         // 4 stages x [A: 128 rows x 128 B][B: NT tokens x 128 B]
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // tiles start on 1024-byte boundaries
    __shared__ __align__(8) uint64_t s_bar[TC_STAGES];
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * TC_ROWS, t0 = blockIdx.y * NT;
    const int nt = min(NT, a.M - t0);
    const int G = a.K >> 6, GP = G >> 1;
    const int ntiles = a.N >> 4;
    if (tid == 0) { for (int i = 0; i < TC_STAGES; ++i) mbar_init(&s_bar[i], 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"((uint32_t)NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem;
    const int T = (row0 >> 4) + warp;                                  // this warp's tile
    const bool tvalid = T < ntiles;                                    // (the last CTA of a matrix whose rows are not a multiple of 128)
    const int r = lane >> 2;
    int cb = 0;
    bool failed = !tc_mainloop<NT>(smem, s_bar, cb, tmem_base, G, tvalid,
        [&](int g, uint4& wv, uint4& sv) {
            wv = ldg_nc_u4(a.q.wr + ((size_t)T * GP + (g >> 1)) * 64 + (g & 1) * 32 + lane);
            sv = ldg_nc_u4(a.q.sr + ((size_t)T * GP + (g >> 1)) * 8 + r);
        },
        [&](int n) -> const __half* { return n < nt ? a.x + (size_t)(t0 + n) * a.ldx : nullptr; });
    failed = __syncthreads_or(failed ? 1 : 0) != 0;
    if (failed && a.err && tid == 0) atomicOr(a.err, 1u);
    if (!failed) {
        // accumulator lane = weight row of the CTA; warps w and w + 4 share a lane quarter and split the token columns
        const int row = row0 + (warp & 3) * 32 + lane;
        const int cbeg = (warp >> 2) * (NT / 2);
        for (int c0 = cbeg; c0 < cbeg + NT / 2; c0 += 32) {
            if (c0 >= nt) break;
            uint32_t dreg[32];
            tmem_ld32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)c0, dreg);
            if (row < a.N) {
#pragma unroll
                for (int n = 0; n < 32; ++n) {
                    if (c0 + n < nt) {
                        const size_t idx = (size_t)(t0 + c0 + n) * a.ldy + row;
                        __half val = f2h(__uint_as_float(dreg[n]));
                        if (a.add_to_y) val = hadd_rn(a.y[idx], val);
                        a.y[idx] = val;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)NT) : "memory");
}

template <int NT>
static int launch_gemm_tc_t(const GemmTcArgs& a, cudaStream_t st) {
    constexpr size_t smem = (size_t)TC_STAGES * (TC_ROWS * 128 + NT * 128) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(k_gemm_umma<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        configured = true;
    }
    dim3 grid((unsigned)((a.N + TC_ROWS - 1) / TC_ROWS), (unsigned)((a.M + NT - 1) / NT));
    k_gemm_umma<NT><<<grid, TC_THREADS, smem, st>>>(a);
    return (int)cudaGetLastError();
}

int launch_gemm_tc(const Q4R& q, int N, int K, int M, const __half* x, int ldx, __half* y, int ldy, bool add_to_y, unsigned* err, cudaStream_t st) {
    if (N % 16 || K % 256) return -1;
    GemmTcArgs a{q, N, K, M, x, ldx, y, ldy, add_to_y ? 1 : 0, err};
    // the token tile is a scheduling choice only: a token's column never interacts with another's
    return M <= 64 ? launch_gemm_tc_t<64>(a, st) : launch_gemm_tc_t<256>(a, st);
}

// ================================================================================ grouped experts (prefill mode)
// Routed + shared experts of a prompt chunk on the same tensor-core pipeline: a work item is (expert slot, block of up to 64
// of its rows, 128 weight rows = 8 tiles); the block's rows are gathered through the pair lists into the B stage, the
// expert's weights are dequantised once per 64 rows.  Items are numbered slot-major, weight-row group fastest; persistent
// CTAs walk them.  gate/up: the epilogue applies SwiGLU to (gate row r, up row r) of a paired tile -- they sit 8
// accumulator lanes apart -- and stores the SwiGLU rows in natural order; down: the pair's output row.
// Prefill-mode numerics (dequantised fp16 weights, one f32 accumulator per output over the whole K); a token's column
// never interacts with another's, so the result does not depend on which rows share a block.
constexpr int XT_NT = 64;
template <bool DOWN>
__global__ void __launch_bounds__(TC_THREADS, 2) k_expert_umma(ExpertArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];         // 4 stages x [A 16 KB][B 8 KB]
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int NT = XT_NT;
    __shared__ __align__(8) uint64_t s_bar[TC_STAGES];
    __shared__ uint32_t s_tmem;
    __shared__ int s_base[260];
    __shared__ int s_srow[NT], s_dst[NT];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2;
    const int K = DOWN ? a.I : a.H, G = K >> 6, GP = G >> 1;
    const int ntiles = DOWN ? a.H / 16 : a.I / 8;                       // tiles of 16 weight rows per expert
    const int NRT = (ntiles + 7) / 8;                                   // groups of 128 weight rows
    const int npair = a.M * a.topk;
    const int n_active = *a.lists.n_active;
    const int nshared = a.M_shared >= 0 ? a.M_shared : a.M;
    if (warp == 0) {                                                    // (slot, block) prefix, as in k_expert_rows
        int run = 0;
        for (int j0 = 0; j0 <= n_active; j0 += 32) {
            const int j = j0 + lane;
            int nb = 0;
            if (j < n_active) nb = (a.lists.slot_cnt[j] + NT - 1) / NT;
            else if (j == n_active) nb = (nshared + NT - 1) / NT;
            int inc = nb;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const int o = __shfl_up_sync(0xffffffffu, inc, d); if (lane >= d) inc += o; }
            if (j <= n_active) s_base[j] = run + inc - nb;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) s_base[n_active + 1] = run;
    }
    if (tid == 0) { for (int i = 0; i < TC_STAGES; ++i) mbar_init(&s_bar[i], 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"((uint32_t)NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem;
    const int total = s_base[n_active + 1] * NRT;
    int cb = 0;                                                          // commits made so far on each stage's barrier (same in every thread)
    bool failed = false;
    for (int item = blockIdx.x; item < total && !failed; item += gridDim.x) {
        const int sb = item / NRT, rt = item - sb * NRT;
        int lo = 0, hi = n_active;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (s_base[mid] <= sb) lo = mid; else hi = mid - 1; }
        const int j = lo, blk = sb - s_base[j];
        const bool shared = (j == n_active);
        const int cnt = shared ? nshared : a.lists.slot_cnt[j];
        const int e = shared ? 0 : a.lists.slot_expert[j];
        const Q4R& q = DOWN ? (shared ? a.sh_down : a.down) : (shared ? a.sh_gu : a.gu);
        if (tid < NT) {
            const int ridx = blk * NT + tid;
            int dst = -1, srow = -1;
            if (ridx < cnt) {
                if (shared) { dst = npair + ridx; srow = DOWN ? dst : a.shared_row0 + ridx; }
                else { const int pr = a.lists.pairs[a.lists.slot_off[j] + ridx]; dst = pr; srow = DOWN ? pr : pr / a.topk; }
            }
            s_srow[tid] = srow; s_dst[tid] = dst;
        }
        __syncthreads();
        const __half* xbase = DOWN ? a.hbuf : a.p;
        const int tile = rt * 8 + warp;
        const bool tvalid = tile < ntiles;
        const size_t Tt = (size_t)e * ntiles + (tvalid ? tile : 0);
        failed = !tc_mainloop<NT>(smem, s_bar, cb, tmem_base, G, tvalid,
            [&](int g, uint4& wv, uint4& sv) {
                wv = ldg_nc_u4(q.wr + (Tt * GP + (g >> 1)) * 64 + (g & 1) * 32 + lane);
                sv = ldg_nc_u4(q.sr + (Tt * GP + (g >> 1)) * 8 + r);
            },
            [&](int n) -> const __half* { const int srow = s_srow[n]; return srow >= 0 ? xbase + (size_t)srow * K : nullptr; });
        failed = __syncthreads_or(failed ? 1 : 0) != 0;
        if (!failed) {
            const int i = (warp & 3) * 32 + lane;                        // accumulator lane = weight row inside the 128
            const int i16 = i & 15, tl = i >> 4, etile = rt * 8 + tl;
            const int c0 = (warp >> 2) * (NT / 2);                       // warps w and w + 4 split the token columns
            uint32_t dreg[32];
            tmem_ld32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)c0, dreg);
#pragma unroll
            for (int n = 0; n < 32; ++n) {
                const float v = __uint_as_float(dreg[n]);
                const int dst = s_dst[c0 + n];
                if (DOWN) {
                    if (dst >= 0 && etile < ntiles) a.dbuf[(size_t)dst * a.H + (size_t)rt * TC_ROWS + i] = f2h(v);
                } else {
                    const float other = __shfl_xor_sync(0xffffffffu, v, 8);               // the up row of this gate row
                    if (dst >= 0 && etile < ntiles && i16 < 8) a.hbuf[(size_t)dst * a.I + etile * 8 + i16] = swiglu_h(f2h(v), f2h(other));
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();                                                 // accumulator, stages and row lists may be reused
    }
    if (failed && a.err && tid == 0) atomicOr(a.err, 1u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)NT) : "memory");
}
template <bool DOWN>
static bool launch_expert_tc_t(const ExpertArgs& a, cudaStream_t st) {
    const int K = DOWN ? a.I : a.H;
    if (K % 256 || a.ep_pairs_per_rank > 0) return false;              // (expert-parallel calls keep the row kernels)
    constexpr size_t smem = (size_t)TC_STAGES * (TC_ROWS * 128 + XT_NT * 128) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_expert_umma<DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
        configured = true;
    }
    const int grid = 2 * sm_count();                                    // 97 KB of shared memory and 64 TMEM columns per CTA: two fit a multiprocessor
    profile_launch(DOWN ? "k_expert_umma_down" : "k_expert_umma_gateup", st, [&] { k_expert_umma<DOWN><<<grid, TC_THREADS, smem, st>>>(a); return 0; });
    return true;
}
bool launch_expert_tc_gateup(const ExpertArgs& a, cudaStream_t st) { return launch_expert_tc_t<false>(a, st); }
bool launch_expert_tc_down(const ExpertArgs& a, cudaStream_t st) { return launch_expert_tc_t<true>(a, st); }

}  // namespace sl
