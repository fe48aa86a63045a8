// rows_kernels.cu -- the many-row forms of the 4-bit group-64 GEMV family: calls with more than 8 activation rows
// (batched decode, long verify rows, strict-mode prompt chunks).
//
// The one-to-eight-row kernels (kernels.cu) walk the rows in passes of 8 and pay one grid wave, one weight fetch and
// one dequantisation per pass.  Here the weights of a tile are fetched and dequantised ONCE per 8*RG rows and a row's
// arithmetic is kept exactly as in the pass kernels, so every output is bit-identical to what the same row gives
// alone (the batch-invariance rule of the reference, swift/Sources/QwispCore/SeedlessMetalForward.swift:160-185):
//   - per group of 64 inputs the same chain of four m16n8k16 MMAs (an MMA column never mixes with another column);
//   - scale * sum and bias * (sum of the group's activations) accumulated over the 4 groups of a 256-input slice;
//   - slice values added in ascending order starting from 0.
//
//   k_rows_prep      the prologue (plain / RMSNorm / gated RMSNorm) of every row, written once per call: activations in the
//                    paired order the dequantiser produces (0,4,1,5,2,6,3,7 inside every 8) + the per-group sums.
//   k_gemv_rows      dense projection: a CTA of 8 warps = 8 tiles x (8*RG rows); the rows' slice of 256 inputs is staged in
//                    shared memory (cp.async, two buffers) and shared by the warps; each warp streams its tile's slices
//                    from global memory two slices ahead.
//   k_expert_rows    routed + shared experts grouped by expert: persistent CTAs of 16 consumer warps + 1 producer warp.
//                    The producer gathers the rows of the next (expert, row block) into a ring of shared-memory stages with
//                    bulk copies (mbarrier full / empty), the consumers each own one tile over the whole K -- no CTA-wide
//                    barrier between experts, which is what bounded the pass kernels when every expert has one or two rows.
//   k_moe_combine    weighted sum of a row's top-k expert rows in ascending k + shared expert + residual.
#include "kernels.h"
#include "gemv.cuh"
#include "route.cuh"

namespace sl {

// ================================================================================ prologue rows
struct RowsPrepArgs {
    const __half* x; int ldx;            // rows (plain) / residual stream (rmsnorm) / mixer output (gated norm)
    const __half* nw; const float* nw32; // norm weight
    const __half* z; int ldz;            // gate input of the gated norm
    float eps; int K;
    __half* xq; float* sxq;              // out: [M][K] paired order, [M][K/64]
};
// grid (M), K/256 warps: warp = one 256-input chunk of the row (the unit of stage_finish())
template <int PRO>
__global__ void __launch_bounds__(512) k_rows_prep(RowsPrepArgs a) {
    __shared__ float part[16];
    const int row = blockIdx.x, ch = threadIdx.x >> 5, lane = threadIdx.x & 31, chunks = a.K >> 8;
    const int k0 = (ch << 8) + lane * 8;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(a.x + (size_t)row * a.ldx + k0));
    uint4 o;
    if (PRO == PRO_PLAIN) {
        o = v;
    } else if (PRO == PRO_RMSNORM) {
        const float ss = warp_sum(sumsq8(v));
        if (lane == 0) part[ch] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int c = 0; c < chunks; ++c) tot += part[c];
        const float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)a.K), a.eps));
        o = rms_apply8(v, *reinterpret_cast<const uint4*>(a.nw + k0), inv);
    } else {
        const uint4 zv = __ldcg(reinterpret_cast<const uint4*>(a.z + (size_t)row * a.ldz + k0));
        const uint4 wv = *reinterpret_cast<const uint4*>(a.nw + (k0 & 127));
        o = normgate8<PRO>(v, zv, wv, a.nw32, k0, a.eps);
    }
    rows_store(a.xq + (size_t)row * a.K, a.sxq + (size_t)row * (a.K >> 6), k0, o, lane);
}
static void launch_rows_prep_args(int pro, const RowsPrepArgs& a, int M, cudaStream_t st) {
    const unsigned threads = (unsigned)(a.K >> 8) * 32u;
    profile_launch("k_rows_prep", st, [&] {
        if (pro == PRO_PLAIN) k_rows_prep<PRO_PLAIN><<<M, threads, 0, st>>>(a);
        else if (pro == PRO_RMSNORM) k_rows_prep<PRO_RMSNORM><<<M, threads, 0, st>>>(a);
        else if (pro == PRO_NORMGATE) k_rows_prep<PRO_NORMGATE><<<M, threads, 0, st>>>(a);
        else k_rows_prep<PRO_NORMGATE32><<<M, threads, 0, st>>>(a);
        return 0;
    });
}
void launch_rows_prep_plain(const __half* x, int ldx, int M, int K, __half* xq, float* sxq, cudaStream_t st) {
    RowsPrepArgs p{x, ldx, nullptr, nullptr, nullptr, 0, 0.f, K, xq, sxq};
    launch_rows_prep_args(PRO_PLAIN, p, M, st);
}

// ================================================================================ shared compute
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
// Wait of the expert kernel's ring, bounded in TIME (~50 ms): the first wait of a CTA that runs out raises the CTA's
// abort word, and every later wait of that CTA gives up at once, so a stall costs one timeout per CTA, not one per item.
constexpr long long XR_TIMEOUT = 100000000ll;                 // cycles
__device__ __forceinline__ bool xr_wait(uint64_t* bar, uint32_t parity, volatile int* abort_word) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; ++i) if (mbar_try_wait(bar, parity)) return true;
        if (*abort_word) return false;
        if (clock64() - t0 > XR_TIMEOUT) { *abort_word = 1; return false; }
    }
}

// One slice (4 groups of 64 inputs) of a 16-row tile against 8*RG staged rows.
// xs: the slice's activations of staged row 0 (paired order), rows xstride halves apart; sxs: group sums of staged
// row 0 for the slice's 4 groups, rows sxstride floats apart.  acc[q]: (row A, col 2t), (A, 2t+1), (B, 2t), (B, 2t+1)
// of row group q.  The order of operations per column is that of compute_slice_x().
template <int RG>
__device__ __forceinline__ void compute_rows(const SliceRegs& rg, const __half* xs, int xstride, const float* sxs, int sxstride,
                                             int r, int t, float accS[RG][4], float accB[RG][4]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint4 wv = rg.w[g];
        uint32_t a0[4], b0[4], a1[4], b1[4];
        dequant8(wv.x, a0); dequant8(wv.z, b0); dequant8(wv.y, a1); dequant8(wv.w, b1);
        const uint4 sv = rg.sc[g >> 1];
        const uint32_t sa_ba = (g & 1) ? sv.z : sv.x, sb_bb = (g & 1) ? sv.w : sv.y;
        const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&sa_ba));
        const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&sb_bb));
#pragma unroll
        for (int q = 0; q < RG; ++q) {
            const __half* xp = xs + (size_t)(q * 8 + r) * xstride + 64 * g + 16 * t;
            const uint4 X0 = *reinterpret_cast<const uint4*>(xp), X1 = *reinterpret_cast<const uint4*>(xp + 8);
            const float sx0 = sxs[(q * 8 + 2 * t) * sxstride + g], sx1 = sxs[(q * 8 + 2 * t + 1) * sxstride + g];
            float c[4];
            mma_f16_z(c, a0[0], b0[0], a0[1], b0[1], X0.x, X0.y);
            mma_f16(c, a0[2], b0[2], a0[3], b0[3], X0.z, X0.w);
            mma_f16(c, a1[0], b1[0], a1[1], b1[1], X1.x, X1.y);
            mma_f16(c, a1[2], b1[2], a1[3], b1[3], X1.z, X1.w);
            accS[q][0] = fmaf(fa.x, c[0], accS[q][0]); accS[q][1] = fmaf(fa.x, c[1], accS[q][1]);
            accS[q][2] = fmaf(fb.x, c[2], accS[q][2]); accS[q][3] = fmaf(fb.x, c[3], accS[q][3]);
            accB[q][0] = fmaf(fa.y, sx0, accB[q][0]); accB[q][1] = fmaf(fa.y, sx1, accB[q][1]);
            accB[q][2] = fmaf(fb.y, sx0, accB[q][2]); accB[q][3] = fmaf(fb.y, sx1, accB[q][3]);
        }
    }
}
// slice value = scale part + bias part, added to the running total (which starts from 0, as reduce_tiles() does)
template <int RG>
__device__ __forceinline__ void add_slice(float tot[RG][4], const float accS[RG][4], const float accB[RG][4]) {
#pragma unroll
    for (int q = 0; q < RG; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) tot[q][i] = __fadd_rn(tot[q][i], __fadd_rn(accS[q][i], accB[q][i]));
}

// ================================================================================ dense projection
struct RowsDenseArgs {
    Q4R q; int N, K, M;
    const __half* xq; const float* sxq;  // prepared rows
    __half* y; int ldy;
};
constexpr int RD_XS = 256 + 8;           // halves per staged row of one slice (16 bytes of skew: conflict-free B loads)
// grid (ceil(tiles / 8), ceil(M / (8*RG))), 256 threads
template <int EPI, int RG>
__global__ void __launch_bounds__(256, RG == 1 ? 2 : 1) k_gemv_rows(RowsDenseArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int NR = 8 * RG;
    __half* xs = reinterpret_cast<__half*>(smem);                               // [2][NR][RD_XS]
    float* sxs = reinterpret_cast<float*>(smem + (size_t)2 * NR * RD_XS * 2);    // [2][NR][4]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, t = lane & 3;
    const int slices = a.K >> 8, G64 = a.K >> 6, ntiles = a.N >> 4;
    const int tile = blockIdx.x * 8 + warp;
    const bool active = tile < ntiles;
    const int row0 = blockIdx.y * NR, nrows = min(NR, a.M - row0);
    const uint4* wt = a.q.wr + (size_t)tile * q4r_w_uint4(a.K);
    const uint4* stl = a.q.sr + (size_t)tile * q4r_s_uint4(a.K);
    auto stage = [&](int s, int b) {
        __half* xb = xs + (size_t)b * NR * RD_XS;
        for (int i = tid; i < NR * 32; i += 256) {
            const int row = i >> 5, c = i & 31;
            __half* dst = xb + (size_t)row * RD_XS + c * 8;
            if (row < nrows) cp_async16(dst, a.xq + (size_t)(row0 + row) * a.K + s * 256 + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        if (tid < NR) {
            float* dst = sxs + (size_t)(b * NR + tid) * 4;
            if (tid < nrows) cp_async16(dst, a.sxq + (size_t)(row0 + tid) * G64 + s * 4);
            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        cp_async_commit();
    };
    SliceRegs cur, n1, n2;                                    // this slice and the next two (weights stream two slices ahead)
    if (active) { load_slice(cur, wt, stl, 0, lane); if (slices > 1) load_slice(n1, wt, stl, 1, lane); }
    stage(0, 0);
    float tot[RG][4];
#pragma unroll
    for (int q = 0; q < RG; ++q) { tot[q][0] = 0.f; tot[q][1] = 0.f; tot[q][2] = 0.f; tot[q][3] = 0.f; }
#pragma unroll 1
    for (int s = 0; s < slices; ++s) {
        const int b = s & 1;
        if (active && s + 2 < slices) load_slice(n2, wt, stl, s + 2, lane);
        if (s + 1 < slices) { stage(s + 1, b ^ 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        if (active) {
            float accS[RG][4], accB[RG][4];
#pragma unroll
            for (int q = 0; q < RG; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) { accS[q][i] = 0.f; accB[q][i] = 0.f; }
            compute_rows<RG>(cur, xs + (size_t)b * NR * RD_XS, RD_XS, sxs + (size_t)b * NR * 4, 4, r, t, accS, accB);
            add_slice<RG>(tot, accS, accB);
        }
        __syncthreads();                       // the buffer may be refilled by the next iteration's stage()
        cur = n1; n1 = n2;
    }
    if (!active) return;
#pragma unroll
    for (int q = 0; q < RG; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int xrow = q * 8 + 2 * t + (i & 1), wrow = tile * 16 + r + 8 * (i >> 1);
            if (xrow < nrows) {
                const size_t idx = (size_t)(row0 + xrow) * a.ldy + wrow;
                __half val = f2h(tot[q][i]);
                if (EPI == EPI_RESID) val = hadd_rn(a.y[idx], val);
                a.y[idx] = val;
            }
        }
}
template <int EPI, int RG>
static void launch_gemv_rows_t(const RowsDenseArgs& a, cudaStream_t st) {
    const size_t smem = (size_t)2 * 8 * RG * RD_XS * 2 + (size_t)2 * 8 * RG * 4 * 4;
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(k_gemv_rows<EPI, RG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); configured = true; }
    const dim3 grid((unsigned)(((a.N >> 4) + 7) / 8), (unsigned)((a.M + 8 * RG - 1) / (8 * RG)));
    profile_launch(EPI == EPI_RESID ? "k_gemv_rows_outproj" : "k_gemv_rows_inproj", st, [&] { k_gemv_rows<EPI, RG><<<grid, 256, smem, st>>>(a); return 0; });
}
// dense projection of M > 8 rows: prologue rows, then the tile kernel.  Returns false when the shape is not covered.
bool launch_dense_rows(int pro, int epi, const DenseArgs& a, cudaStream_t st) {
    if (!a.xq || !a.sxq || a.K % 256 || a.K > 4096 || a.N % 16 || (epi != EPI_STORE && epi != EPI_RESID)) return false;
    RowsPrepArgs p{a.x, a.ldx, a.nw, a.nw32, a.z, a.ldz, a.eps, a.K, a.xq, a.sxq};
    launch_rows_prep_args(pro, p, a.M, st);
    RowsDenseArgs d{a.q, a.N, a.K, a.M, a.xq, a.sxq, a.y, a.ldy};
    // 32 rows per CTA (weights dequantised once per 32 rows) when that still fills the device, else 8
    const long ctas4 = (long)(((a.N >> 4) + 7) / 8) * ((a.M + 31) / 32);
    const bool rg4 = ctas4 >= sm_count();
    if (epi == EPI_RESID) { if (rg4) launch_gemv_rows_t<EPI_RESID, 4>(d, st); else launch_gemv_rows_t<EPI_RESID, 1>(d, st); }
    else { if (rg4) launch_gemv_rows_t<EPI_STORE, 4>(d, st); else launch_gemv_rows_t<EPI_STORE, 1>(d, st); }
    return true;
}

// ================================================================================ experts
// A work item is (expert slot, block of 8 rows, group of 16 tiles); items are numbered slot-major, tile group fastest, so
// neighbouring CTAs read neighbouring weights and the same rows.  Slot n_active is the shared expert (all rows).
constexpr int XR_CONS = 16;                  // consumer warps = tiles per item
constexpr int XR_THREADS = (XR_CONS + 1) * 32;
struct XrStage {                             // one ring stage in shared memory
    __half* xs;                              // [8][K + 8]
    float* sxs;                              // [8][K/64 + 4]
    float* craw;                             // down: [8][K/8] chunk sums as written by the gate/up kernel
    int* info;                               // [0..7] destination rows (-1: none), [8] expert, [9] shared, [10] tile group
};
template <bool DOWN>
__host__ __device__ inline size_t xr_stage_bytes(int K) {
    size_t b = (size_t)8 * (K + 8) * 2 + (size_t)8 * (K / 64 + 4) * 4 + 16 * 4;
    if (DOWN) b += (size_t)8 * (K / 8) * 4;
    return (b + 15) & ~(size_t)15;
}
template <bool DOWN>
__device__ __forceinline__ XrStage xr_carve(unsigned char* base, int K) {
    XrStage s;
    s.xs = reinterpret_cast<__half*>(base); base += (size_t)8 * (K + 8) * 2;
    s.sxs = reinterpret_cast<float*>(base); base += (size_t)8 * (K / 64 + 4) * 4;
    s.craw = reinterpret_cast<float*>(base); if (DOWN) base += (size_t)8 * (K / 8) * 4;
    s.info = reinterpret_cast<int*>(base);
    return s;
}
// grid: one CTA per multiprocessor; dynamic shared memory: nstages stages
template <bool DOWN>
__global__ void __launch_bounds__(XR_THREADS, 1) k_expert_rows(ExpertArgs a, int nstages) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_base[260];                                  // first (slot, block) index of every slot; [n_active + 1] = total
    __shared__ __align__(8) uint64_t s_full[8], s_empty[8], s_raw[8];
    __shared__ int s_sig; __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, t = lane & 3;
    const int K = DOWN ? a.I : a.H;
    const int slices = K >> 8, G64 = K >> 6, SXS = G64 + 4, XS = K + 8;
    const int ntiles = DOWN ? a.H / 16 : a.I / 8;
    const int NTG = (ntiles + XR_CONS - 1) / XR_CONS;
    const int npair = a.M * a.topk;
    const int n_active = *a.lists.n_active;
    const int nshared = a.M_shared >= 0 ? a.M_shared : a.M;
    const size_t stage_bytes = xr_stage_bytes<DOWN>(K);
    // ---- (slot, block) prefix: warp 0 scans the slot counts in chunks of 32
    if (warp == 0) {
        int run = 0;
        for (int j0 = 0; j0 <= n_active; j0 += 32) {
            const int j = j0 + lane;
            int nb = 0;
            if (j < n_active) nb = (a.lists.slot_cnt[j] + 7) >> 3;
            else if (j == n_active) nb = (nshared + 7) >> 3;
            int inc = nb;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const int o = __shfl_up_sync(0xffffffffu, inc, d); if (lane >= d) inc += o; }
            if (j <= n_active) s_base[j] = run + inc - nb;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) s_base[n_active + 1] = run;
    }
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < nstages; ++i) { mbar_init(&s_full[i], DOWN ? 1 : 8); mbar_init(&s_empty[i], XR_CONS); mbar_init(&s_raw[i], 8); }
        mbar_fence_init();
    }
    __syncthreads();
    const int total = s_base[n_active + 1] * NTG;
    // (slot, block) index -> slot: the last j with s_base[j] <= sb
    auto slot_of = [&](int sb) {
        int lo = 0, hi = n_active;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (s_base[mid] <= sb) lo = mid; else hi = mid - 1; }
        return lo;
    };
    bool failed = false;
    unsigned fail_code = 0;          // which wait ran out: 16 producer/empty, 32 producer/chunk sums, 64 consumer/full
    if (warp == XR_CONS) {
        // ------------------------------------------------------------ producer
        int k = 0;
        for (int item = blockIdx.x; item < total; item += gridDim.x, ++k) {
            const int stg = k % nstages, use = k / nstages;
            const XrStage S = xr_carve<DOWN>(smem + (size_t)stg * stage_bytes, K);
            if (use > 0 && !xr_wait(&s_empty[stg], (uint32_t)((use - 1) & 1), &s_abort)) { failed = true; fail_code |= 16u; break; }
            const int sb = item / NTG, tg = item - sb * NTG;
            const int j = slot_of(sb), blk = sb - s_base[j];
            const bool shared = (j == n_active);
            const int cnt = shared ? nshared : a.lists.slot_cnt[j];
            if (lane < 8) {
                const int ridx = blk * 8 + lane;
                int dst = -1, srow = 0;
                if (ridx < cnt) {
                    if (shared) { dst = npair + ridx; srow = DOWN ? dst : a.shared_row0 + ridx; }
                    else { const int pr = a.lists.pairs[a.lists.slot_off[j] + ridx]; dst = pr; srow = DOWN ? pr : pr / a.topk; }
                }
                S.info[lane] = dst;
                if (lane == 0) { S.info[8] = shared ? 0 : a.lists.slot_expert[j]; S.info[9] = shared ? 1 : 0; S.info[10] = tg; }
                uint64_t* bar = DOWN ? &s_raw[stg] : &s_full[stg];
                if (dst >= 0) {
                    const __half* xsrc = (DOWN ? a.hbuf : a.xq) + (size_t)srow * K;
                    if (DOWN) {
                        mbar_expect_tx(bar, (uint32_t)(K * 2 + (K / 8) * 4));
                        bulk_g2s(S.xs + (size_t)lane * XS, xsrc, (uint32_t)K * 2, bar);
                        bulk_g2s(S.craw + (size_t)lane * (K / 8), a.csum + (size_t)srow * (K / 8), (uint32_t)(K / 8) * 4, bar);
                    } else {
                        mbar_expect_tx(bar, (uint32_t)(K * 2 + G64 * 4));
                        bulk_g2s(S.xs + (size_t)lane * XS, xsrc, (uint32_t)K * 2, bar);
                        bulk_g2s(S.sxs + (size_t)lane * SXS, a.sxq + (size_t)srow * G64, (uint32_t)G64 * 4, bar);
                    }
                } else {
                    mbar_arrive(bar);
                }
            }
            if (DOWN) {
                // group sums from the chunk sums: eight chunk sums combined in the butterfly order of rows_store()
                if (!xr_wait(&s_raw[stg], (uint32_t)(use & 1), &s_abort)) { failed = true; fail_code |= 32u; break; }
                for (int i = lane; i < 8 * G64; i += 32) {
                    const int row = i / G64, g = i - row * G64;
                    const float* c = S.craw + (size_t)row * (K / 8) + g * 8;
                    const float4 lo = *reinterpret_cast<const float4*>(c), hi = *reinterpret_cast<const float4*>(c + 4);
                    const float e = __fadd_rn(__fadd_rn(lo.x, hi.x), __fadd_rn(lo.z, hi.z));       // (s0 + s4) + (s2 + s6)
                    const float o = __fadd_rn(__fadd_rn(lo.y, hi.y), __fadd_rn(lo.w, hi.w));       // (s1 + s5) + (s3 + s7)
                    S.sxs[(size_t)row * SXS + g] = __fadd_rn(e, o);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_full[stg]);
            }
        }
    } else {
        // ------------------------------------------------------------ consumers: warp = one tile of the item's group
        const Q4R& qr = DOWN ? a.down : a.gu;
        const Q4R& qs = DOWN ? a.sh_down : a.sh_gu;
        const size_t wstep = q4r_w_uint4(K), sstep = q4r_s_uint4(K);
        auto tile_ptrs = [&](int item, const uint4*& wt, const uint4*& stl, bool& valid) {
            const int sb = item / NTG, tg = item - sb * NTG;
            const int j = slot_of(sb);
            const bool shared = (j == n_active);
            const int tile = tg * XR_CONS + warp;
            valid = tile < ntiles;
            const Q4R& q = shared ? qs : qr;
            const size_t T = (size_t)(shared ? 0 : a.lists.slot_expert[j]) * ntiles + (valid ? tile : 0);
            wt = q.wr + T * wstep; stl = q.sr + T * sstep;
        };
        SliceRegs cur, nxt;
        const uint4 *wt = nullptr, *stl = nullptr, *wt_n = nullptr, *stl_n = nullptr;
        bool valid = false, valid_n = false;
        if ((int)blockIdx.x < total) { tile_ptrs(blockIdx.x, wt, stl, valid); if (valid) load_slice(cur, wt, stl, 0, lane); }
        int k = 0;
        for (int item = blockIdx.x; item < total; item += gridDim.x, ++k) {
            const int stg = k % nstages, use = k / nstages;
            const XrStage S = xr_carve<DOWN>(smem + (size_t)stg * stage_bytes, K);
            const int item_n = item + gridDim.x;
            if (item_n < total) tile_ptrs(item_n, wt_n, stl_n, valid_n); else valid_n = false;
            if (!xr_wait(&s_full[stg], (uint32_t)(use & 1), &s_abort)) { failed = true; fail_code |= 64u; break; }
            float tot[1][4] = {{0.f, 0.f, 0.f, 0.f}};
#pragma unroll 1
            for (int s = 0; s < slices; ++s) {
                if (s + 1 < slices) { if (valid) load_slice(nxt, wt, stl, s + 1, lane); }
                else if (valid_n) load_slice(nxt, wt_n, stl_n, 0, lane);
                if (valid) {
                    float accS[1][4] = {{0.f, 0.f, 0.f, 0.f}}, accB[1][4] = {{0.f, 0.f, 0.f, 0.f}};
                    compute_rows<1>(cur, S.xs + s * 256, XS, S.sxs + s * 4, SXS, r, t, accS, accB);
                    add_slice<1>(tot, accS, accB);
                }
                cur = nxt;
            }
            if (valid) {
                const int tile = S.info[10] * XR_CONS + warp;
                if (DOWN) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int dst = S.info[2 * t + (i & 1)];
                        if (dst >= 0) {
                            __half* rowp = a.dbuf + (size_t)dst * a.H;
                            if (a.ep_pairs_per_rank > 0 && dst < npair) {       // routed pair in expert-parallel mode: the owner's buffer
                                const int own = dst / a.ep_pairs_per_rank;
                                rowp = a.peer_dbuf[own] + (size_t)(dst - own * a.ep_pairs_per_rank) * a.H;
                            }
                            rowp[tile * 16 + r + 8 * (i >> 1)] = f2h(tot[0][i]);
                        }
                    }
                } else {
                    // SwiGLU of (gate row r, up row r) per column; the 8 outputs of a column (lanes with the same t) form one
                    // 8-chunk of the down projection's input: stored in the paired order with its chunk sum
#pragma unroll
                    for (int jc = 0; jc < 2; ++jc) {
                        const __half hv = swiglu_h(f2h(tot[0][jc]), f2h(tot[0][2 + jc]));
                        const unsigned hb = __half_as_ushort(hv);
                        unsigned v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = __shfl_sync(0xffffffffu, hb, i * 4 + t);
                        const int dst = S.info[2 * t + jc];
                        if (r == 0 && dst >= 0) {
                            const uint4 nat = make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
                            const uint4 prd = make_uint4(v[0] | (v[4] << 16), v[1] | (v[5] << 16), v[2] | (v[6] << 16), v[3] | (v[7] << 16));
                            *reinterpret_cast<uint4*>(a.hbuf + (size_t)dst * a.I + tile * 8) = prd;
                            a.csum[(size_t)dst * (a.I / 8) + tile] = sum8_f32(nat);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[stg]);
            wt = wt_n; stl = stl_n; valid = valid_n;
        }
    }
    if (failed && a.err && lane == 0) atomicOr(a.err, fail_code | (DOWN ? 8u : 4u));
    __syncthreads();
    if (s_abort) {                             // bulk copies this CTA started may still be landing in its shared memory: outlast them
        const long long t0 = clock64();
        while (clock64() - t0 < 200000ll) { }
    }
    if (DOWN && a.ep_sig.world > 0) {
        // expert-parallel: every CTA makes its peer stores visible system-wide and draws a ticket; the last one raises this
        // rank's combine flag at every peer
        __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            const unsigned ticket = atomicAdd(a.ep_sig.ticket, 1u);
            s_sig = (ticket == gridDim.x - 1) ? 1 : 0;
            if (s_sig) *a.ep_sig.ticket = 0u;
        }
        __syncthreads();
        if (s_sig && tid < a.ep_sig.world)
            st_release_sys(a.ep_sig.flags[tid] + 8 + a.ep_sig.rank, ep_seq(a.ep_sig.ctr, a.ep_sig.layer, 1));
    }
}
template <bool DOWN>
static bool launch_expert_rows_t(const ExpertArgs& a, cudaStream_t st) {
    const int K = DOWN ? a.I : a.H;
    if (K % 256 || K > 4096 || !a.csum || (!DOWN && (!a.xq || !a.sxq))) return false;
    const size_t sb = xr_stage_bytes<DOWN>(K);
    int nstages = (int)((size_t)(190 * 1024) / sb);
    if (nstages > 8) nstages = 8;
    if (nstages < 2) return false;
    const size_t smem = sb * nstages;
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(k_expert_rows<DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); configured = true; }
    const int grid = sm_count();
    profile_launch(DOWN ? "k_expert_rows_down" : "k_expert_rows_gateup", st, [&] { k_expert_rows<DOWN><<<grid, XR_THREADS, smem, st>>>(a, nstages); return 0; });
    return true;
}
bool launch_expert_rows_gateup(const ExpertArgs& a, cudaStream_t st) { return launch_expert_rows_t<false>(a, st); }
bool launch_expert_rows_down(const ExpertArgs& a, cudaStream_t st) { return launch_expert_rows_t<true>(a, st); }

// ================================================================================ router for many rows
// k_router_rows   logits of all rows: a CTA keeps 8 router rows (or the shared gate) in registers and walks the row
//                 groups of 8, whose normed rows arrive in shared memory by cp.async two groups ahead of their use.
//                 The dot product is the one of k_moe_router (lane l owns 8 consecutive inputs of every 256-wide block,
//                 sequential f32 accumulate, butterfly over the lanes), so the logits are the same bits.
// k_route_rows    one warp per row: top-k + gates (route_row_warp); the last CTA groups the (row, k) pairs by expert with
//                 a parallel scan (or, expert-parallel, sends rows and indices to every rank).
// Input rows are already normed (k_final_norm), so no CTA repeats the norm.
template <bool Q8>
__global__ void __launch_bounds__(256, 2) k_router_rows(RouterArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];                   // [2][8][H] halves
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nblk = a.H >> 8;
    const bool tail = (blockIdx.x == gridDim.x - 1);
    const int e = blockIdx.x * 8 + warp;
    const bool wvalid = tail ? (warp == 0) : (e < a.E);
    uint4 wreg[16]; uint2 qreg[16]; __half2 sbreg[16];
    if constexpr (Q8) {
        const uint8_t* qrow = tail ? a.sg_q8 : (a.router_q8 + (size_t)e * a.H);
        const __half* srow = tail ? a.sg_qs : (a.router_qs + (size_t)e * (a.H >> 6));
        const __half* brow = tail ? a.sg_qb : (a.router_qb + (size_t)e * (a.H >> 6));
#pragma unroll
        for (int kb = 0; kb < 16; ++kb) {
            const bool ok = wvalid && kb < nblk;
            qreg[kb] = ok ? *reinterpret_cast<const uint2*>(qrow + kb * 256 + lane * 8) : make_uint2(0, 0);
            sbreg[kb] = ok ? __halves2half2(srow[kb * 4 + (lane >> 3)], brow[kb * 4 + (lane >> 3)]) : __halves2half2(f2h(0.f), f2h(0.f));
        }
    } else {
        const __half* wrow = tail ? a.shared_gate : (a.router + (size_t)e * a.H);
#pragma unroll
        for (int kb = 0; kb < 16; ++kb)
            wreg[kb] = (wvalid && kb < nblk) ? *reinterpret_cast<const uint4*>(wrow + kb * 256 + lane * 8) : make_uint4(0, 0, 0, 0);
    }
    const int ngroups = (a.M + 7) >> 3;
    auto stage = [&](int rg, int b) {
        __half* dst = reinterpret_cast<__half*>(smem) + (size_t)b * 8 * a.H;
        const int mr = min(8, a.M - rg * 8);
        for (int i = tid; i < mr * (a.H >> 3); i += 256) cp_async16(dst + (size_t)i * 8, a.h + (size_t)rg * 8 * a.ldh + (size_t)(i / (a.H >> 3)) * a.ldh + (size_t)(i % (a.H >> 3)) * 8);
        cp_async_commit();
    };
    int it = 0;
    if ((int)blockIdx.y < ngroups) stage(blockIdx.y, 0);
    for (int rg = blockIdx.y; rg < ngroups; rg += gridDim.y, ++it) {
        const int b = it & 1;
        if (rg + (int)gridDim.y < ngroups) { stage(rg + gridDim.y, b ^ 1); cp_async_wait<1>(); } else cp_async_wait<0>();
        __syncthreads();
        const __half* ps = reinterpret_cast<const __half*>(smem) + (size_t)b * 8 * a.H;
        const int m0 = rg * 8, mr = min(8, a.M - m0);
        if (wvalid) {
            for (int c = 0; c < mr; ++c) {
                const __half* xrow = ps + (size_t)c * a.H;
                float acc = 0.f;
#pragma unroll
                for (int kb = 0; kb < 16; ++kb) {
                    if (kb < nblk) {
                        const uint4 xv = *reinterpret_cast<const uint4*>(xrow + kb * 256 + lane * 8);
                        const __half* xh = reinterpret_cast<const __half*>(&xv);
                        if constexpr (Q8) {
                            float sum = 0.f, accum = 0.f;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float xf = h2f(xh[i]);
                                const unsigned q = ((i < 4 ? qreg[kb].x : qreg[kb].y) >> (8 * (i & 3))) & 0xffu;
                                sum = __fadd_rn(sum, xf);
                                accum = fmaf(xf, (float)q, accum);
                            }
                            const float2 sb = __half22float2(sbreg[kb]);
                            acc = __fadd_rn(acc, __fadd_rn(__fmul_rn(sb.x, accum), __fmul_rn(sum, sb.y)));
                        } else {
                            const __half* wh = reinterpret_cast<const __half*>(&wreg[kb]);
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc = fmaf(h2f(xh[i]), h2f(wh[i]), acc);
                        }
                    }
                }
                const float d = warp_sum(acc);
                if (lane == 0) { if (tail) a.sgl[m0 + c] = f2h(d); else a.logits[(size_t)(m0 + c) * a.E + e] = f2h(d); }
            }
        }
        __syncthreads();                       // the buffer is refilled by the next iteration's stage()
    }
}
// grid (ceil(M / 8)), 256 threads: one warp per row.  Expert-parallel: grid (M), one row per CTA.
__global__ void __launch_bounds__(256) k_route_rows(RouterArgs a) {
    __shared__ float s_route[8][512 + 32];
    __shared__ int s_cnt[256], s_off[256], s_slot[256], s_cur[256], s_wsum[8], s_wact[8];
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (a.epd.sig.world > 0) {
        // expert-parallel (grid = M, one row per CTA): warp 0 routes the row, then warp w stores the normed row and its
        // routing indices into rank w's gather buffers over peer memory; the CTA that finishes last raises this rank's
        // dispatch flag at every rank.  The pair lists are built from the gathered indices by k_ep_lists.
        const EpSignal& sg = a.epd.sig;
        const int m = blockIdx.x;
        if (warp == 0) route_row_warp(a.logits + (size_t)m * a.E, a.E, a.topk, a.inds + m * a.topk, a.scores + m * a.topk, s_route[0], lane);
        __syncthreads();
        for (int d = warp; d < sg.world; d += 8) {
            if (!a.ep_rows_sent) {
                const uint4* src = reinterpret_cast<const uint4*>(a.p + (size_t)m * a.H);
                uint4* dst = reinterpret_cast<uint4*>(a.epd.pbuf[d] + ((size_t)sg.rank * a.M + m) * a.H);
                for (int i = lane; i < a.H / 8; i += 32) dst[i] = __ldcg(src + i);
            }
            int* di = a.epd.ibuf[d] + ((size_t)sg.rank * a.M + m) * a.topk;
            if (lane < a.topk) di[lane] = a.inds[m * a.topk + lane];
        }
        __threadfence_system();
        __syncthreads();
        if (tid == 0) { const unsigned ticket = atomicAdd(a.counter, 1u); s_last = (ticket == gridDim.x - 1) ? 1 : 0; }
        __syncthreads();
        if (!s_last) return;
        __threadfence_system();
        if (tid == 0) *a.counter = 0u;
        if (tid < sg.world) st_release_sys(sg.flags[tid] + sg.rank, ep_seq(sg.ctr, sg.layer, 0));
        return;
    }
    const int m = blockIdx.x * 8 + warp;
    if (m < a.M) route_row_warp(a.logits + (size_t)m * a.E, a.E, a.topk, a.inds + m * a.topk, a.scores + m * a.topk, s_route[warp], lane);
    __threadfence();
    __syncthreads();
    if (tid == 0) { const unsigned ticket = atomicAdd(a.counter, 1u); s_last = (ticket == gridDim.x - 1) ? 1 : 0; }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *a.counter = 0u;
    // ---- pairs grouped by expert: counts, then slot numbers and offsets by a block scan (thread = expert)
    s_cnt[tid] = 0; s_cur[tid] = 0;
    __syncthreads();
    const int npairs = a.M * a.topk;
    for (int i = tid; i < npairs; i += 256) atomicAdd(&s_cnt[__ldcg(a.inds + i)], 1);
    __syncthreads();
    const int cnt = (tid < a.E) ? s_cnt[tid] : 0, act = cnt > 0 ? 1 : 0;
    int isum = cnt, iact = act;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int o1 = __shfl_up_sync(0xffffffffu, isum, d), o2 = __shfl_up_sync(0xffffffffu, iact, d);
        if (lane >= d) { isum += o1; iact += o2; }
    }
    if (lane == 31) { s_wsum[warp] = isum; s_wact[warp] = iact; }
    __syncthreads();
    int bsum = 0, bact = 0;
    for (int w = 0; w < warp; ++w) { bsum += s_wsum[w]; bact += s_wact[w]; }
    const int off = bsum + isum - cnt, slot = bact + iact - act;
    s_off[tid] = off; s_slot[tid] = slot;
    if (act) { a.lists.slot_expert[slot] = tid; a.lists.slot_off[slot] = off; a.lists.slot_cnt[slot] = cnt; }
    if (tid == 255) *a.lists.n_active = slot + act;
    __syncthreads();
    for (int i = tid; i < npairs; i += 256) {
        const int ex = __ldcg(a.inds + i);
        const int pos = atomicAdd(&s_cur[ex], 1);
        a.lists.pairs[s_off[ex] + pos] = i;
    }
}
// Prefill mode: the fp16 router logits as a small tensor-core GEMM (mma.sync m16n8k16, f32 accumulators): a CTA of 4 warps
// computes 64 rows x 64 experts, K in chunks of 64 through two cp.async buffers (16-byte pieces swizzled by the row).
// Not the bit pattern of the strict router (the f32 sums run in MMA order), but a row's logits depend on that row only
// and K is walked in a fixed order, so they do not depend on how a prompt is cut into calls.  The shared-gate logit is a
// plain warp dot (the strict order) done by the CTAs of the first expert tile.
__device__ __forceinline__ void rt_ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ __half* rt_at(__half* base, int row, int chunk) { return base + row * 64 + ((chunk ^ (row & 7)) << 3); }   // rows of 64 halves
__global__ void __launch_bounds__(128) k_router_mma(RouterArgs a) {
    __shared__ __align__(128) __half As[2][64 * 64], Bs[2][64 * 64];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * 64, e0 = blockIdx.y * 64;
    const int rows = min(64, a.M - m0), cols = min(64, a.E - e0);
    auto stage = [&](int kc, int b) {
        for (int i = tid; i < 64 * 8; i += 128) {
            const int r = i >> 3, c = i & 7;
            if (r < rows) cp_async16(rt_at(As[b], r, c), a.h + (size_t)(m0 + r) * a.ldh + kc * 64 + c * 8);
            else *reinterpret_cast<uint4*>(rt_at(As[b], r, c)) = make_uint4(0, 0, 0, 0);
            if (r < cols) cp_async16(rt_at(Bs[b], r, c), a.router + (size_t)(e0 + r) * a.H + kc * 64 + c * 8);
            else *reinterpret_cast<uint4*>(rt_at(Bs[b], r, c)) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) { acc[n][0] = 0.f; acc[n][1] = 0.f; acc[n][2] = 0.f; acc[n][3] = 0.f; }
    const int nk = a.H >> 6;
    stage(0, 0);
    for (int kc = 0; kc < nk; ++kc) {
        const int b = kc & 1;
        if (kc + 1 < nk) { stage(kc + 1, b ^ 1); cp_async_wait<1>(); } else cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t a0, a1, a2, a3;
            rt_ldsm_x4(a0, a1, a2, a3, rt_at(As[b], warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;
                const int mi = lane >> 3;
                rt_ldsm_x4(b0, b1, b2, b3, rt_at(Bs[b], (np * 2 + (mi >> 1)) * 8 + (lane & 7), ks * 2 + (mi & 1)));
                mma_f16(acc[np * 2], a0, a1, a2, a3, b0, b1);
                mma_f16(acc[np * 2 + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = warp * 16 + (lane >> 2) + 8 * (i >> 1), c = n * 8 + 2 * (lane & 3) + (i & 1);
            if (r < rows && c < cols) a.logits[(size_t)(m0 + r) * a.E + e0 + c] = f2h(acc[n][i]);
        }
    if (blockIdx.y == 0) {                     // shared-gate logit of the CTA's rows: lane l owns 8 inputs of every 256-wide block
        for (int r = warp; r < rows; r += 4) {
            const __half* xrow = a.h + (size_t)(m0 + r) * a.ldh;
            float s = 0.f;
            for (int kb = 0; kb < (a.H >> 8); ++kb) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xrow + kb * 256 + lane * 8);
                const uint4 wv = *reinterpret_cast<const uint4*>(a.shared_gate + kb * 256 + lane * 8);
                const __half* xh = reinterpret_cast<const __half*>(&xv);
                const __half* wh = reinterpret_cast<const __half*>(&wv);
#pragma unroll
                for (int i = 0; i < 8; ++i) s = fmaf(h2f(xh[i]), h2f(wh[i]), s);
            }
            s = warp_sum(s);
            if (lane == 0) a.sgl[m0 + r] = f2h(s);
        }
    }
}
// prefill mode, fp16 router: logits on the tensor cores, then the routing / pair-list kernel.  false: not covered.
bool launch_router_mma(const RouterArgs& a, cudaStream_t st) {
    if (a.E > 256 || a.H % 256 || a.norm_w || a.router_q8 || a.sg_q8) return false;
    const dim3 grid((unsigned)((a.M + 63) / 64), (unsigned)((a.E + 63) / 64));
    profile_launch("k_router_mma", st, [&] { k_router_mma<<<grid, 128, 0, st>>>(a); return 0; });
    profile_launch("k_route_rows", st, [&] { k_route_rows<<<a.epd.sig.world > 0 ? a.M : (a.M + 7) / 8, 256, 0, st>>>(a); return 0; });
    return true;
}

// rows already normed in a.h (ldh); E <= 256.  Returns false when the shape is not covered.
bool launch_router_rows(const RouterArgs& a, cudaStream_t st) {
    if (a.E > 256 || a.H % 256 || a.H > 4096 || a.norm_w) return false;
    const size_t smem = (size_t)2 * 8 * a.H * 2;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(k_router_rows<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        cudaFuncSetAttribute(k_router_rows<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        configured = true;
    }
    const int ngroups = (a.M + 7) / 8;
    const int gx = (a.E + 7) / 8 + 1;
    int gy = (2 * sm_count() + gx - 1) / gx; if (gy > ngroups) gy = ngroups; if (gy < 1) gy = 1;
    const dim3 grid((unsigned)gx, (unsigned)gy);
    const bool q8 = a.router_q8 != nullptr;
    profile_launch("k_router_rows", st, [&] {
        if (q8) k_router_rows<true><<<grid, 256, smem, st>>>(a); else k_router_rows<false><<<grid, 256, smem, st>>>(a);
        return 0;
    });
    const int route_grid = a.epd.sig.world > 0 ? a.M : ngroups;
    profile_launch("k_route_rows", st, [&] { k_route_rows<<<route_grid, 256, 0, st>>>(a); return 0; });
    return true;
}

// ================================================================================ combine
// grid (M), 256 threads:
// out/resid[m] (+)= sum_k fp16(d[m*topk + k] * score[m,k]) (ascending k) + sigmoid(sgl[m]) * shared[m]
// (swift/Sources/QwispCore/SeedlessFusedVerify.swift:462-484, SeedlessMetalForward.swift:1024-1028)
__global__ void __launch_bounds__(256) k_moe_combine(const __half* dbuf, const __half* shared_rows, const __half* scores, const __half* sgl,
                                                     int H, int topk, __half* resid, __half* out) {
    const int m = blockIdx.x;
    for (int n = threadIdx.x; n < H; n += blockDim.x) {
        __half acc = f2h(0.0f);
        for (int k = 0; k < topk; ++k)
            acc = hadd_rn(acc, hmul_rn(__ldcg(dbuf + (size_t)(m * topk + k) * H + n), scores[m * topk + k]));
        const __half res = hadd_rn(acc, hmul_rn(sigmoid_h(sgl[m]), __ldcg(shared_rows + (size_t)m * H + n)));
        if (resid) resid[(size_t)m * H + n] = hadd_rn(resid[(size_t)m * H + n], res);
        else out[(size_t)m * H + n] = res;
    }
}
void launch_moe_combine(const __half* dbuf, const __half* shared_rows, const __half* scores, const __half* sgl, int M, int H, int topk,
                        __half* resid, __half* out, cudaStream_t st) {
    profile_launch("k_moe_combine", st, [&] { k_moe_combine<<<M, 256, 0, st>>>(dbuf, shared_rows, scores, sgl, H, topk, resid, out); return 0; });
}

}  // namespace sl
