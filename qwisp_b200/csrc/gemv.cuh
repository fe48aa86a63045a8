// gemv.cuh -- 4-bit group-64 GEMV family ("F1": decode / verify rows, M-invariant per row).
//
// y[m, n] = sum_k x[m, k] * (scale[n, k/64] * q[n, k] + bias[n, k/64]),  q = nibble k%8 of
// word w[n, k/8] (low nibble first) -- the MLX affine layout of the reference
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:219-221, 238-310).
//
// B200 formulation.  HBM-bound, and at one activation row the legacy f16 tensor path would
// itself become a bottleneck, so the goal is few instructions AND few MMAs per weight nibble:
//   * a 4-bit value q in the low half of a byte, read as an fp8 e4m3 number, is exactly q * 2^-9
//     (q < 8 are subnormals, q >= 8 normals with exponent field 1), so nibbles become tensor-core
//     operands with one AND (and one shift for the odd ones): no conversion, no table;
//   * mma.sync m16n8k32 e4m3 x e4m3 -> f32 consumes 16 weight rows x 32 inputs per instruction;
//   * an fp16 activation is split exactly into three e4m3 terms x = x1 + x2/16 + x3/256 (each
//     term carries 4 significant bits of the residual); the three terms sit in three of the eight
//     MMA columns, so one instruction yields all three partial products and an MMA pass serves
//     two activation rows (columns 0-2 and 3-5).  Products are exact, accumulation is f32;
//   * per group of 64 inputs: acc += scale * C + bias * sum(x): two FMAs per group and output
//     instead of per element (the algebra the reference uses, SeedlessMetalForward.swift:249-258);
//   * a warp owns 16 weight rows x 256 inputs (one "slice" = 4 groups); weights are read in the
//     fragment-major layout below with 128-bit coalesced loads;
//   * each row's result is independent of how many rows share the call (columns of an MMA do not
//     interact) and slices are summed in ascending order whatever the CTA organisation.
#pragma once
#include <cuda_fp8.h>
#include "common.cuh"

namespace sl {

enum { PRO_PLAIN = 0, PRO_RMSNORM = 1, PRO_NORMGATE = 2 };
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_ARGMAX = 3 };

constexpr int ROWS_PER_PASS = 2;     // activation rows per MMA pass (3 term columns each)

struct XStage {
    unsigned char* xs;   // [rows][3 terms][K + 64] e4m3 bytes in fragment order
    float* sxs;          // [K/64][2] per-group sums of x (bias term)
    float* part;         // [2][16] scratch for the rmsnorm prologue
    int stride;          // K + 64 (bytes) between terms
};

// Sum of 8 consecutive activations the way the reference's GEMV forms its bias term: groups of
// four are added in fp16 (each add rounded), the fp16 partial sums are then added in f32
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:238-247).  Matching this keeps fp16
// outputs identical to the CPU restatement except at rare rounding boundaries.
__device__ __forceinline__ float sum8_f32(uint4 v) {
    const __half* h = reinterpret_cast<const __half*>(&v);
    __half a = hadd_rn(hadd_rn(hadd_rn(h[0], h[1]), h[2]), h[3]);
    __half b = hadd_rn(hadd_rn(hadd_rn(h[4], h[5]), h[6]), h[7]);
    return h2f(a) + h2f(b);
}
// fp16 pair -> e4m3 pair (round to nearest, saturating) and back
__device__ __forceinline__ uint32_t to_e4m3x2(__half2 v) {
    return (uint32_t)__nv_cvt_halfraw2_to_fp8x2(static_cast<__half2_raw>(v), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ __half2 from_e4m3x2(uint32_t e) {
    return __half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)e, __NV_E4M3));
}
// 8 consecutive fp16 values -> three 8-byte e4m3 terms in fragment order (x0,x2,x4,x6, x1,x3,x5,x7);
// x = t1 + t2/16 + t3/256 exactly (every residual is exactly representable in fp16)
__device__ __forceinline__ void split_terms8(uint4 v, uint2 out[3]) {
    const __half2 k16 = __floats2half2_rn(16.f, 16.f);
    __half2 r[4];
    const __half2* hv = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = hv[i];
#pragma unroll
    for (int term = 0; term < 3; ++term) {
        uint32_t e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            e[i] = to_e4m3x2(r[i]);
            if (term < 2) r[i] = __hmul2(__hsub2(r[i], from_e4m3x2(e[i])), k16);
        }
        uint32_t A = e[0] | (e[1] << 16), B = e[2] | (e[3] << 16);      // bytes x0,x1,x2,x3 / x4,x5,x6,x7
        out[term].x = __byte_perm(A, B, 0x6420);
        out[term].y = __byte_perm(A, B, 0x7531);
    }
}
// lane holds 8 consecutive activations of pass-row `col` starting at k0 (multiple of 8): write
// the staged terms and accumulate the group sum (8 consecutive lanes cover one group of 64)
__device__ __forceinline__ void store_staged(const XStage& st, int col, int k0, uint4 v, int lane) {
    float s = sum8_f32(v);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 7) == 0) st.sxs[(k0 >> 6) * 2 + col] = s;
    uint2 tm[3];
    split_terms8(v, tm);
#pragma unroll
    for (int term = 0; term < 3; ++term)
        *reinterpret_cast<uint2*>(st.xs + (size_t)(col * 3 + term) * st.stride + k0) = tm[term];
}

// ---- prologues: stage `mr` (<= ROWS_PER_PASS) activation rows of width K ----
// Split in two so that a kernel can put its few activation loads in flight BEFORE its many weight
// loads (an SM serves its memory requests in order: activations queued behind 100+ KB of weights
// would arrive last and nothing could be computed while the weights stream in), and only then
// wait for them.  A warp owns 256-wide chunks; with two rows of K <= 4096 there are at most two per
// warp of a 16-warp CTA (four per warp of an 8-warp CTA are not supported: K <= 2048 there).
struct StageSrc {
    const __half* x; int ldx;        // rows (plain) / residual stream (rmsnorm) / y (normgate)
    const int* rows;                 // optional row list (shared memory), else rows row0, row0+1
    const __half* nw;                // norm weight
    const __half* z; int ldz;        // gate input of the gated norm
    float eps;
};
struct StageRegs { uint4 a[2], b[2], c[2]; };

template <int PRO>
__device__ __forceinline__ void stage_issue(StageRegs& sr, const StageSrc& s, int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8, units = mr * chunks;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        int u = warp + j * nw;
        if (u < units) {
            int col = (u >= chunks) ? 1 : 0, ch = u - col * chunks, k0 = ch * 256 + lane * 8;
            int row = s.rows ? s.rows[col] : row0 + col;
            sr.a[j] = __ldcg(reinterpret_cast<const uint4*>(s.x + (size_t)row * s.ldx + k0));
            if (PRO == PRO_RMSNORM) sr.b[j] = *reinterpret_cast<const uint4*>(s.nw + k0);
            if (PRO == PRO_NORMGATE) {
                sr.b[j] = *reinterpret_cast<const uint4*>(s.nw + (k0 & 127));
                sr.c[j] = __ldcg(reinterpret_cast<const uint4*>(s.z + (size_t)row * s.ldz + k0));
            }
        }
    }
}
__device__ __forceinline__ uint4 rms_apply8(uint4 v, uint4 wv, float inv) {
    const __half* hv = reinterpret_cast<const __half*>(&v);
    const __half* wh = reinterpret_cast<const __half*>(&wv);
    uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int i = 0; i < 8; ++i) oh[i] = hmul_rn(wh[i], f2h(__fmul_rn(h2f(hv[i]), inv)));
    return o;
}
__device__ __forceinline__ float sumsq8(uint4 v) {
    const __half2* hh = reinterpret_cast<const __half2*>(&v);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(hh[i]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
    return ss;
}
// RMSNorm: x = w * fp16(h * inv), inv = rsqrt(mean(h^2) + eps) (SeedlessMetalForward.swift:800-827).
// Gated RMSNorm of the GDN out-projection, per head of 128:
// x = fp16(silu_f32(z) * float(w * fp16(y * inv))) (SeedlessFusedVerify.swift:803-813).
// Contains one __syncthreads() for PRO_RMSNORM; the caller synchronises before reading xs.
template <int PRO>
__device__ __forceinline__ void stage_finish(const StageRegs& sr, const XStage& st, const StageSrc& s, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8, units = mr * chunks;
    if (PRO == PRO_RMSNORM) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            int u = warp + j * nw;
            if (u < units) {
                int col = (u >= chunks) ? 1 : 0, ch = u - col * chunks;
                float ss = warp_sum(sumsq8(sr.a[j]));
                if (lane == 0) st.part[col * 16 + ch] = ss;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        int u = warp + j * nw;
        if (u < units) {
            int col = (u >= chunks) ? 1 : 0, ch = u - col * chunks, k0 = ch * 256 + lane * 8;
            uint4 o;
            if (PRO == PRO_PLAIN) {
                o = sr.a[j];
            } else if (PRO == PRO_RMSNORM) {
                float tot = 0.f;
                for (int c = 0; c < chunks; ++c) tot += st.part[col * 16 + c];
                float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), s.eps));
                o = rms_apply8(sr.a[j], sr.b[j], inv);
            } else {
                const __half* yh = reinterpret_cast<const __half*>(&sr.a[j]);
                const __half* zh = reinterpret_cast<const __half*>(&sr.c[j]);
                const __half* wh = reinterpret_cast<const __half*>(&sr.b[j]);
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) { float f = h2f(yh[i]); ss = fmaf(f, f, ss); }
                ss = half_warp_sum(ss);                       // 16 lanes per head of 128
                float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), s.eps));
                __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float nrm = h2f(hmul_rn(wh[i], f2h(__fmul_rn(h2f(yh[i]), inv))));
                    float zf = h2f(zh[i]);
                    oh[i] = f2h(__fmul_rn(__fmul_rn(zf, sigmoid_f(zf)), nrm));
                }
            }
            store_staged(st, col, k0, o, lane);
        }
    }
}
// generic (any number of chunks per warp) versions used by the persistent head kernel
__device__ __forceinline__ void stage_plain(const XStage& st, const __half* x, int ldx, int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8;
    for (int u = warp; u < mr * chunks; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;
        uint4 v = __ldcg(reinterpret_cast<const uint4*>(x + (size_t)(row0 + col) * ldx + k0));
        store_staged(st, col, k0, v, lane);
    }
}
__device__ __forceinline__ void stage_rmsnorm(const XStage& st, const __half* h, int ldh, const __half* w, float eps,
                                              int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8, units = mr * chunks;
    for (int u = warp; u < units; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;
        uint4 v = __ldcg(reinterpret_cast<const uint4*>(h + (size_t)(row0 + col) * ldh + k0));
        float ss = warp_sum(sumsq8(v));
        if (lane == 0) st.part[col * 16 + ch] = ss;
    }
    __syncthreads();
    for (int u = warp; u < units; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;
        float tot = 0.f;
        for (int c = 0; c < chunks; ++c) tot += st.part[col * 16 + c];
        float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), eps));
        uint4 v = __ldcg(reinterpret_cast<const uint4*>(h + (size_t)(row0 + col) * ldh + k0));
        uint4 wv = *reinterpret_cast<const uint4*>(w + k0);
        store_staged(st, col, k0, rms_apply8(v, wv, inv), lane);
    }
}

// ---- L2 prefetch of weights a LATER kernel will read: keeps HBM streaming while this kernel and
//      the kernel boundary are busy with latency-bound work.  Ranges are cut into 8 KB pieces;
//      piece c is issued by CTA c % n_cta (flat CTA index), one piece per thread.
struct PfList { const void* p[6]; unsigned bytes[6]; };
__device__ __forceinline__ void prefetch_ranges(const PfList& pf, int cta, int n_cta) {
    int base = 0;
#pragma unroll
    for (int i = 0; i < 6; ++i) {
        if (pf.p[i] == nullptr || pf.bytes[i] == 0) continue;
        int pieces = (int)((pf.bytes[i] + 8191u) >> 13);
        // pieces of this range owned by this CTA: c with (base + c) % n_cta == cta
        int first = ((cta - base) % n_cta + n_cta) % n_cta;
        int c = first + (int)threadIdx.x * n_cta;
        if (c < pieces) {
            unsigned off = (unsigned)c << 13;
            unsigned len = pf.bytes[i] - off; if (len > 8192u) len = 8192u;
            len &= ~15u;
            if (len) prefetch_l2_bulk(reinterpret_cast<const char*>(pf.p[i]) + off, len);
        }
        base = (base + pieces) % n_cta;
    }
}

// ---- fragment-major weight layout ("repacked" once at load time from the MLX affine layout) ----
// A tile is 16 weight rows: A_0..A_7 and B_0..B_7 (for a dense matrix rows 16T..16T+7 and 16T+8..16T+15;
// for the fused gate/up projection 8 gate rows and the 8 up rows of the same outputs).  K = 64*G
// groups, taken in pairs (GP = G/2).  For tile T and group pair gp:
//   Wr: uint4 [T][gp][2 groups][32 lanes]   lane (r = lane/4, t = lane%4), group g = 2gp+gi:
//         { A_r word 8g+2t, A_r word 8g+2t+1, B_r word 8g+2t, B_r word 8g+2t+1 }   (word = 8 nibbles of the MLX layout)
//   Sr: uint4 [T][gp][8 rows r]             fp16 { sA(g0), bA(g0), sB(g0), bB(g0), sA(g1), bA(g1), sB(g1), bB(g1) }
// so a warp's loads are 512 contiguous bytes of nibbles per group and 128 bytes of scales per pair,
// each lane exactly the 16 inputs x 2 rows its tensor-core fragments need.  Same 0.5625 B/weight.
struct Q4R { const uint4* wr = nullptr; const uint4* sr = nullptr; int tiles = 0; int K = 0; };

__host__ __device__ inline size_t q4r_w_uint4(int K) { return (size_t)(K / 128) * 64; }   // per tile
__host__ __device__ inline size_t q4r_s_uint4(int K) { return (size_t)(K / 128) * 8; }    // per tile

// ---- weight slice (256 inputs = 4 groups = 2 pairs) held in registers ----
struct SliceRegs { uint4 w[4]; uint4 sc[2]; };

__device__ __forceinline__ void load_slice(SliceRegs& rg, const uint4* wr_tile, const uint4* sr_tile, int slice, int lane) {
    const uint4* wp = wr_tile + (size_t)slice * 128 + lane;
    rg.w[0] = ldg_nc_u4(wp); rg.w[1] = ldg_nc_u4(wp + 32); rg.w[2] = ldg_nc_u4(wp + 64); rg.w[3] = ldg_nc_u4(wp + 96);
    const uint4* sp = sr_tile + (size_t)slice * 16 + (lane >> 2);
    rg.sc[0] = ldg_nc_u4(sp); rg.sc[1] = ldg_nc_u4(sp + 8);
}

// (not volatile: pure functions of their operands, so the compiler may interleave independent groups)
__device__ __forceinline__ void mma_e4m3(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// first MMA of a group: the accumulator starts from zero without spending registers on it
__device__ __forceinline__ void mma_e4m3_z(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// One slice (4 groups) of a 16-row tile against the staged rows.  MMA column n = lane/4 carries
// pass-row n/3, term n%3 (columns 6,7 unused).  accS/accB [4]: (row A, col 2t), (row A, col 2t+1),
// (row B, col 2t), (row B, col 2t+1); the bias term is added once per pass-row, in its term-0 column.
__device__ __forceinline__ void compute_slice(const SliceRegs& r, const XStage& st, int slice, int n, int t, int mr,
                                              float accS[4], float accB[4]) {
    const bool col_active = (n < 3 * mr);
    const unsigned char* xp = st.xs + (size_t)n * st.stride + slice * 256 + 16 * t;     // n = row*3 + term
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 X = make_uint4(0, 0, 0, 0);
        if (col_active) X = *reinterpret_cast<const uint4*>(xp + 64 * g);
        const uint4 wv = r.w[g];
        float c[4];
        mma_e4m3_z(c, wv.x & 0x0f0f0f0fu, wv.z & 0x0f0f0f0fu, (wv.x >> 4) & 0x0f0f0f0fu, (wv.z >> 4) & 0x0f0f0f0fu, X.x, X.y);
        mma_e4m3(c, wv.y & 0x0f0f0f0fu, wv.w & 0x0f0f0f0fu, (wv.y >> 4) & 0x0f0f0f0fu, (wv.w >> 4) & 0x0f0f0f0fu, X.z, X.w);
        const float2 sx2 = *reinterpret_cast<const float2*>(st.sxs + (slice * 4 + g) * 2);
        const float sx0 = (t == 0) ? sx2.x : 0.f;       // column 0 = row 0 term 0
        const float sx1 = (t == 1) ? sx2.y : 0.f;       // column 3 = row 1 term 0
        const uint4 sv = r.sc[g >> 1];
        const uint32_t sa_ba = (g & 1) ? sv.z : sv.x, sb_bb = (g & 1) ? sv.w : sv.y;
        float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&sa_ba));    // (scale A, bias A)
        float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&sb_bb));    // (scale B, bias B)
        accS[0] = fmaf(fa.x, c[0], accS[0]); accS[1] = fmaf(fa.x, c[1], accS[1]);
        accS[2] = fmaf(fb.x, c[2], accS[2]); accS[3] = fmaf(fb.x, c[3], accS[3]);
        accB[0] = fmaf(fa.y, sx0, accB[0]); accB[1] = fmaf(fa.y, sx1, accB[1]);
        accB[2] = fmaf(fb.y, sx0, accB[2]); accB[3] = fmaf(fb.y, sx1, accB[3]);
    }
}
// undo the operand scales: nibbles carry 2^-9, term k of the activation carries 16^k
__device__ __forceinline__ void finish_acc4(const float accS[4], const float accB[4], int t, float v[4]) {
    const int m0 = (2 * t) % 3, m1 = (2 * t + 1) % 3;
    const float k0 = (m0 == 0) ? 512.f : ((m0 == 1) ? 32.f : 2.f);
    const float k1 = (m1 == 0) ? 512.f : ((m1 == 1) ? 32.f : 2.f);
    v[0] = fmaf(accS[0], k0, accB[0]);
    v[1] = fmaf(accS[1], k1, accB[1]);
    v[2] = fmaf(accS[2], k0, accB[2]);
    v[3] = fmaf(accS[3], k1, accB[3]);
}
// value of pass-row j (0/1) of weight row `row` from the reduced 16x8 tile: the three term columns in order
__device__ __forceinline__ float tile_value(const float* fin_tile, int row, int j) {
    const float* p = fin_tile + row * 8 + 3 * j;
    return (p[0] + p[1]) + p[2];
}

// ---- CTA organisation of the split GEMV ----
// A tile is 16 weight rows; its K/256 slices are shared by WPT warps of SPW slices each, and a CTA
// holds TPC tiles.  Every slice's value is kept separate and the slices are summed in ascending
// order whatever the split, so the split is a pure scheduling choice: results do not depend on it.
struct GemvPlan { int upw, tpc, nw, lg_slices; };
// K/256 must be a power of two (K = 256, 512, ... 4096).  A unit is one slice of one tile; a CTA of
// 16 warps takes UPW units per warp (unit u = warp + 16*i -> tile u >> lg_slices, slice u & (slices-1)),
// i.e. TPC = 16*UPW/slices whole tiles.  UPW grows (to at most 3) until `groups` independent
// problems of `ntiles` tiles fit one wave of 148 CTAs.
__host__ __device__ inline GemvPlan gemv_plan(int K, int ntiles, int groups) {
    GemvPlan p;
    int slices = K >> 8;
    p.lg_slices = 0; while ((1 << p.lg_slices) < slices) ++p.lg_slices;
    p.nw = 16;
    long long units = (long long)ntiles * slices * groups;
    int upw = (int)((units + 148 * 16 - 1) / (148 * 16));
    if (upw < 1) upw = 1;
    if (upw > 3) upw = 3;
    while ((p.nw * upw) % slices) ++upw;          // whole tiles per CTA (slices <= 16 divides 16)
    p.upw = upw;
    p.tpc = p.nw * upw / slices;
    return p;
}

// element i of a warp's 128 partials is lane = i>>2, ci = i&3: row = (lane>>2) + 8*(ci>>1), col = 2*(lane&3) + (ci&1)
__device__ __forceinline__ void store_partial(float* red, int slot, int lane, const float v[4]) {
    *reinterpret_cast<float4*>(red + slot * 128 + lane * 4) = make_float4(v[0], v[1], v[2], v[3]);
}
// red [tpc][slices][128] -> fin [tpc][row*8 + col]; call between two __syncthreads()
__device__ __forceinline__ void reduce_tiles(const float* red, float* fin, int tpc, int slices) {
    for (int i = threadIdx.x; i < tpc * 128; i += blockDim.x) {
        int tl = i >> 7, j = i & 127;
        float acc = 0.f;
        for (int sidx = 0; sidx < slices; ++sidx) acc += red[(tl * slices + sidx) * 128 + j];
        int l = j >> 2, ci = j & 3;
        int row = (l >> 2) + 8 * (ci >> 1), col = 2 * (l & 3) + (ci & 1);
        fin[tl * 128 + row * 8 + col] = acc;
    }
}

// dynamic shared memory carve-up shared by host (size) and device (pointers)
struct GemvSmem {
    __host__ __device__ static size_t bytes(int rows, int K, int nred, int tpc) {
        size_t xs = (size_t)rows * 3 * (K + 64);
        return xs + (size_t)(K / 64) * 2 * 4 + 2 * 16 * 4 + (size_t)nred * 128 * 4 + (size_t)tpc * 128 * 4 + 128;
    }
    __device__ static void carve(unsigned char* base, int rows, int K, int nred, int tpc, XStage& st, float*& red, float*& fin, int*& misc) {
        size_t xs = (size_t)rows * 3 * (K + 64);
        st.xs = base;
        st.sxs = reinterpret_cast<float*>(base + xs);
        st.part = st.sxs + (K / 64) * 2;
        red = st.part + 2 * 16;
        fin = red + nred * 128;
        misc = reinterpret_cast<int*>(fin + tpc * 128);      // 32 ints
        st.stride = K + 64;
    }
};

}  // namespace sl
