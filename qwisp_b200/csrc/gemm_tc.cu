// gemm_tc.cu -- 4-bit group-64 GEMM for many activation rows ("F2": prefill chunks) on the 5th-generation
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
// A CTA of 128 threads owns 128 weight rows (8 tiles of the fragment-major layout) and NT activation rows (64 or 256).
// Two shared-memory stages alternate over the K groups of 64 inputs:
//   fill   every thread dequantises two fragment registers (16 nibbles of two weight rows, scale and bias applied with
//          one fp16x2 multiply-add per pair) into the A stage -- K-major rows of 128 bytes, 128-byte swizzle, the 8 halves
//          of a 16-byte chunk in the pair order (0,4,1,5,2,6,3,7) the one-logic-op dequantiser produces -- and copies
//          NT x 64 activations into the B stage in the same order, so no permutation is spent; operands travel global ->
//          registers -> shared memory in two register sets, a group's loads being issued a whole iteration ahead;
//   issue  fence.proxy.async + barrier; one thread issues four MMAs (M=128, N=NT, K=16) that accumulate into the NT
//          TMEM columns and commits them to the stage's mbarrier; the CTA goes straight on to fill the other stage,
//          waiting (bounded) on a stage's mbarrier only before it overwrites it.
// Two CTAs fit a multiprocessor (97 KB of shared memory, 256 TMEM columns each), so one CTA's fill overlaps the other's MMAs.
// (An unswizzled operand layout ran the same MMAs about five times slower.)
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
// fragment registers of one 16-row tile (wv: nibbles of rows A_r / B_r, sv: their scales and biases for the pair of
// groups) -> fp16 weights in the A stage
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
            uint32_t d[4];
            dequant8(words[wi], d);
            const __half2 sc = (wi < 2) ? sA2 : sB2, bi = (wi < 2) ? bA2 : bB2;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o[wi]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 wq = __hfma2(*reinterpret_cast<const __half2*>(&d[j]), sc, bi);
                ow[j] = *reinterpret_cast<const uint32_t*>(&wq);
            }
        }
    }
    const int rowA = tl * 16 + r;                                     // row A_r of the tile; B_r is 8 rows further (the next atom)
    *reinterpret_cast<uint4*>(tc_at(sA, rowA, 2 * t)) = o[0];
    *reinterpret_cast<uint4*>(tc_at(sA, rowA, 2 * t + 1)) = o[1];
    *reinterpret_cast<uint4*>(tc_at(sA, rowA + 8, 2 * t)) = o[2];
    *reinterpret_cast<uint4*>(tc_at(sA, rowA + 8, 2 * t + 1)) = o[3];
}
// piece idx of the B stage: token = 8 * (idx / 64) + idx % 8, chunk = (idx / 8) % 8 -- the 8 lanes of a quarter warp store
// into the 8 rows of one atom (distinct swizzled chunks: no bank conflict) and read 4 x 64 contiguous bytes per token row
__device__ __forceinline__ void tc_piece(int idx, int& n, int& c) { n = ((idx >> 6) << 3) + (idx & 7); c = (idx >> 3) & 7; }
template <int NT>
__device__ __forceinline__ void tc_store_B(unsigned char* sB, int tid, const uint4* xv) {
#pragma unroll
    for (int h = 0; h < NT * 8 / 128; ++h) {
        int n, c; tc_piece(tid + 128 * h, n, c);
        const uint4 v = xv[h];
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410); o.y = __byte_perm(v.x, v.z, 0x7632);
        o.z = __byte_perm(v.y, v.w, 0x5410); o.w = __byte_perm(v.y, v.w, 0x7632);
        *reinterpret_cast<uint4*>(tc_at(sB, n, c)) = o;
    }
}
// one thread: four MMAs of K = 16 (two 16-byte chunks each) accumulating into the NT columns, then the commit
template <int NT>
__device__ __forceinline__ void tc_issue(unsigned char* sA, unsigned char* sB, uint32_t tmem_base, uint32_t idesc, bool first, uint64_t* bar) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        const uint64_t da = umma_desc_sw128(sA + ks * 32), db = umma_desc_sw128(sB + ks * 32);      // 16 halves further along K
        umma_f16(tmem_base, da, db, idesc, (!first || ks > 0) ? 1u : 0u);
    }
    umma_commit(bar);
}

struct GemmTcArgs {
    Q4R q; int N, K, M;
    const __half* x; int ldx;
    __half* y; int ldy;
    int add_to_y;                    // y += result (residual) instead of y = result
    unsigned* err;
};

template <int NT>
__global__ void __launch_bounds__(128) k_gemm_umma(GemmTcArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];         // 2 stages x [A: 128 rows x 128 B][B: NT tokens x 128 B]
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // tiles start on 1024-byte boundaries
    constexpr int A_BYTES = 8 * TC_ROWS * 16, B_BYTES = 8 * NT * 16, STAGE = A_BYTES + B_BYTES;
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * TC_ROWS, t0 = blockIdx.y * NT;
    const int nt = min(NT, a.M - t0);
    const int G = a.K >> 6, GP = G >> 1;
    const int ntiles = a.N >> 4;
    if (tid == 0) { mbar_init(&s_bar[0], 1); mbar_init(&s_bar[1], 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"((uint32_t)NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);   // f32 accumulate, f16 x f16, K-major both
    bool failed = false;
    // Operands of a K group travel global -> registers -> shared memory.  All of a group's loads are issued together, and
    // the next group's loads are issued before this group's MMAs, so one round trip to L2 is in flight per group instead
    // of one per load.
    constexpr int NB = NT * 8 / 128;                                       // 16-byte activation pieces per thread and group
    const int r = lane >> 2, t = lane & 3;
    struct Regs { uint4 wv[2], sv[2], xv[NB]; };
    Regs ra, rb;                                                           // two register sets: a group's loads have a whole iteration to land
    bool tvalid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) tvalid[h] = ((row0 >> 4) + warp + 4 * h) < ntiles;   // (the last CTA of a matrix whose rows are not a multiple of 128)
    auto load_group = [&](Regs& R, int g) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int T = (row0 >> 4) + warp + 4 * h;
            if (tvalid[h]) {
                R.wv[h] = ldg_nc_u4(a.q.wr + ((size_t)T * GP + (g >> 1)) * 64 + (g & 1) * 32 + lane);
                R.sv[h] = ldg_nc_u4(a.q.sr + ((size_t)T * GP + (g >> 1)) * 8 + r);
            }
        }
#pragma unroll
        for (int h = 0; h < NB; ++h) {
            int n, c; tc_piece(tid + 128 * h, n, c);
            R.xv[h] = (n < nt) ? __ldcg(reinterpret_cast<const uint4*>(a.x + (size_t)(t0 + n) * a.ldx + g * 64 + c * 8)) : make_uint4(0, 0, 0, 0);
        }
    };
    auto process = [&](const Regs& R, int g) {
        const int s = g & 1, use = g >> 1;
        unsigned char* sA = smem + (size_t)s * STAGE;
        unsigned char* sB = sA + A_BYTES;
        // the MMAs that read this stage two groups ago must be done before it is overwritten
        if (use > 0 && !tc_wait(&s_bar[s], (uint32_t)((use - 1) & 1))) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int h = 0; h < 2; ++h) tc_dequant_A(sA, warp + 4 * h, r, t, g, R.wv[h], R.sv[h], tvalid[h]);
        tc_store_B<NT>(sB, tid, R.xv);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) tc_issue<NT>(sA, sB, tmem_base, idesc, g == 0, &s_bar[s]);
    };
    load_group(ra, 0);
    for (int g = 0; g < G; g += 2) {                                       // G is even (K is a multiple of 256)
        load_group(rb, g + 1);
        process(ra, g);
        if (g + 2 < G) load_group(ra, g + 2);
        process(rb, g + 1);
    }
    // the last commit covers every MMA issued before it
    if (!tc_wait(&s_bar[(G - 1) & 1], (uint32_t)(((G - 1) >> 1) & 1))) failed = true;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    failed = __syncthreads_or(failed ? 1 : 0) != 0;
    if (failed && a.err && tid == 0) atomicOr(a.err, 1u);
    if (!failed) {
        const int row = row0 + tid;
        for (int c0 = 0; c0 < NT; c0 += 32) {
            if (c0 >= nt) break;
            uint32_t dreg[32];
            tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, dreg);
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
    constexpr size_t smem = 2 * (8 * TC_ROWS * 16 + 8 * NT * 16) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(k_gemm_umma<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        configured = true;
    }
    dim3 grid((unsigned)((a.N + TC_ROWS - 1) / TC_ROWS), (unsigned)((a.M + NT - 1) / NT));
    k_gemm_umma<NT><<<grid, 128, smem, st>>>(a);
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
__global__ void __launch_bounds__(128) k_expert_umma(ExpertArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];         // 2 stages x [A 16 KB][B 8 KB]
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // tiles start on 1024-byte boundaries
    constexpr int NT = XT_NT, A_BYTES = 8 * TC_ROWS * 16, B_BYTES = 8 * NT * 16, STAGE = A_BYTES + B_BYTES, NB = NT * 8 / 128;
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_base[260];
    __shared__ int s_srow[NT], s_dst[NT];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, t = lane & 3;
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
    if (tid == 0) { mbar_init(&s_bar[0], 1); mbar_init(&s_bar[1], 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"((uint32_t)NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);
    const int total = s_base[n_active + 1] * NRT;
    int commits[2] = {0, 0};                                             // commits made so far on each stage's barrier (same in every thread)
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
        struct Regs { uint4 wv[2], sv[2], xv[NB]; };
        Regs ra, rb;
        bool tvalid[2];
        size_t Tt[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) { const int tile = rt * 8 + warp + 4 * h; tvalid[h] = tile < ntiles; Tt[h] = (size_t)e * ntiles + (tvalid[h] ? tile : 0); }
        auto load_group = [&](Regs& R, int g) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (tvalid[h]) {
                    R.wv[h] = ldg_nc_u4(q.wr + (Tt[h] * GP + (g >> 1)) * 64 + (g & 1) * 32 + lane);
                    R.sv[h] = ldg_nc_u4(q.sr + (Tt[h] * GP + (g >> 1)) * 8 + r);
                }
#pragma unroll
            for (int h = 0; h < NB; ++h) {
                int n, c; tc_piece(tid + 128 * h, n, c);
                const int srow = s_srow[n];
                R.xv[h] = (srow >= 0) ? __ldcg(reinterpret_cast<const uint4*>(xbase + (size_t)srow * K + g * 64 + c * 8)) : make_uint4(0, 0, 0, 0);
            }
        };
        auto process = [&](const Regs& R, int g) {
            const int s = g & 1;
            unsigned char* sA = smem + (size_t)s * STAGE;
            unsigned char* sB = sA + A_BYTES;
            // the MMAs that read this stage two groups ago (in this item) must be done before it is overwritten
            if (g >= 2 && !tc_wait(&s_bar[s], (uint32_t)((commits[s] - 1) & 1))) failed = true;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < 2; ++h) tc_dequant_A(sA, warp + 4 * h, r, t, g, R.wv[h], R.sv[h], tvalid[h]);
            tc_store_B<NT>(sB, tid, R.xv);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if (tid == 0) tc_issue<NT>(sA, sB, tmem_base, idesc, g == 0, &s_bar[s]);
            commits[s] += 1;
        };
        load_group(ra, 0);
        for (int g = 0; g < G; g += 2) {
            load_group(rb, g + 1);
            process(ra, g);
            if (g + 2 < G) load_group(ra, g + 2);
            process(rb, g + 1);
        }
        {   // the last commit covers every MMA of the item
            const int s = (G - 1) & 1;
            if (!tc_wait(&s_bar[s], (uint32_t)((commits[s] - 1) & 1))) failed = true;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        failed = __syncthreads_or(failed ? 1 : 0) != 0;
        if (!failed) {
            const int i16 = tid & 15, tl = tid >> 4, tile = rt * 8 + tl;
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t dreg[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, dreg);
#pragma unroll
                for (int n = 0; n < 32; ++n) {
                    const float v = __uint_as_float(dreg[n]);
                    const int dst = s_dst[c0 + n];
                    if (DOWN) {
                        if (dst >= 0 && tile < ntiles) a.dbuf[(size_t)dst * a.H + (size_t)rt * TC_ROWS + tid] = f2h(v);
                    } else {
                        const float other = __shfl_xor_sync(0xffffffffu, v, 8);               // the up row of this gate row
                        if (dst >= 0 && tile < ntiles && i16 < 8) a.hbuf[(size_t)dst * a.I + tile * 8 + i16] = swiglu_h(f2h(v), f2h(other));
                    }
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
    constexpr size_t smem = 2 * (8 * TC_ROWS * 16 + 8 * XT_NT * 16) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_expert_umma<DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
        configured = true;
    }
    const int grid = 4 * sm_count();                                    // 48 KB of shared memory and 64 TMEM columns per CTA: four fit a multiprocessor
    profile_launch(DOWN ? "k_expert_umma_down" : "k_expert_umma_gateup", st, [&] { k_expert_umma<DOWN><<<grid, 128, smem, st>>>(a); return 0; });
    return true;
}
bool launch_expert_tc_gateup(const ExpertArgs& a, cudaStream_t st) { return launch_expert_tc_t<false>(a, st); }
bool launch_expert_tc_down(const ExpertArgs& a, cudaStream_t st) { return launch_expert_tc_t<true>(a, st); }

}  // namespace sl
