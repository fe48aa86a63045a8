// gemv.cuh -- 4-bit group-64 GEMV family ("F1": decode / verify rows, M-invariant per row).
//
// y[m, n] = sum_k x[m, k] * (scale[n, k/64] * q[n, k] + bias[n, k/64]),  q = nibble k%8 of
// word w[n, k/8] (low nibble first) -- the MLX affine layout of the reference
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:219-221, 238-310).
//
// B200 formulation.  HBM-bound; the work per weight nibble on the SM must stay small, and it is
// the integer/logic pipe (half rate) that saturates first:
//   * nibbles become exact fp16 integers in registers with one logic op per PAIR of weights:
//     (w & 0x000F000F) | 0x64006400 is the fp16x2 {1024+q0, 1024+q4}, (w & 0x00F000F0) | 0x64006400
//     is {1024+16*q1, 1024+16*q5}; the same two masks on w >> 8 give q2,q6 and q3,q7.  One fp16x2
//     subtract (or multiply-add with 1/16, -64) per register removes offset and factor exactly;
//     that runs on the FMA pipe, which has room.  (An fp8 e4m3 operand path was measured first:
//     on this part mma.sync with e4m3 operands is executed by converting every operand register
//     to fp16, 12 conversions per instruction on the logic pipe, so it is slower, not faster.)
//   * mma.sync m16n8k16 f16 x f16 -> f32: 16 weight rows x 16 inputs per instruction, the eight
//     columns are eight activation rows, so one pass serves up to 8 rows.  Products are exact
//     (4-bit integer x fp16), accumulation is f32;
//   * the pairing (q_i, q_{i+4}) is matched by storing each 8 activations in shared memory in the
//     order 0,4,1,5,2,6,3,7, so one 128-bit shared load is the B operand of two instructions;
//   * per group of 64 inputs: acc += scale * C + bias * sum(x): two FMAs per group and output
//     instead of per element (the algebra the reference uses, SeedlessMetalForward.swift:249-258);
//   * a warp owns 16 weight rows x 256 inputs (one "slice" = 4 groups); weights are read in the
//     fragment-major layout below, which arrives in shared memory by bulk asynchronous copies;
//   * each row's result is independent of how many rows share the call (columns of an MMA do not
//     interact) and slices are summed in ascending order whatever the CTA organisation.
#pragma once
#include "common.cuh"

namespace sl {

enum { PRO_PLAIN = 0, PRO_RMSNORM = 1, PRO_NORMGATE = 2, PRO_NORMGATE32 = 3 };   // NORMGATE32: gated norm with an f32 weight
__host__ __device__ constexpr bool pro_is_normgate(int pro) { return pro == PRO_NORMGATE || pro == PRO_NORMGATE32; }
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_ARGMAX = 3 };

constexpr int ROWS_PER_PASS = 8;     // activation rows per MMA pass (the 8 columns of m16n8k16)

struct XStage {
    __half* xs;          // [rows][stride] fp16, every 8 consecutive inputs stored as 0,4,1,5,2,6,3,7
    float* sxs;          // [K/64][8] per-group sums of x (bias term)
    float* part;         // [8][16] scratch for the rmsnorm prologue
    int stride;          // K + 8 (halves) between rows: 16 bytes of skew keeps the B loads conflict-free
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
// lane holds 8 consecutive activations of pass-row `col` starting at k0 (multiple of 8): write
// them in the paired order and accumulate the group sum (8 consecutive lanes cover one group of 64)
__device__ __forceinline__ void store_staged(const XStage& st, int col, int k0, uint4 v, int lane) {
    float s = sum8_f32(v);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 7) == 0) st.sxs[(k0 >> 6) * 8 + col] = s;
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);       // (x0, x4)
    o.y = __byte_perm(v.x, v.z, 0x7632);       // (x1, x5)
    o.z = __byte_perm(v.y, v.w, 0x5410);       // (x2, x6)
    o.w = __byte_perm(v.y, v.w, 0x7632);       // (x3, x7)
    *reinterpret_cast<uint4*>(st.xs + (size_t)col * st.stride + k0) = o;
}

// The same for the many-row kernels, whose prepared rows live in global memory ([M][K] paired order, [M][K/64] sums):
// lane holds the 8 prologue'd activations (row, k0 .. k0+7): paired-order store + group sum (8 lanes = one group),
// the arithmetic of store_staged()
__device__ __forceinline__ void rows_store(__half* xq_row, float* sx_row, int k0, uint4 v, int lane) {
    float s = sum8_f32(v);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 7) == 0) sx_row[k0 >> 6] = s;
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    *reinterpret_cast<uint4*>(xq_row + k0) = o;
}
// ---- prologues: stage `mr` (<= ROWS_PER_PASS) activation rows of width K ----
// A warp owns 256-wide chunks (unit u = row * chunks + chunk, units u = warp, warp + nw, ...).
// The first two units of a warp are requested by stage_issue and held in registers, so a kernel
// can put those loads in flight early and do other set-up before it needs them; further units
// (more than two rows, or K = 4096 with two) are loaded where they are used.
struct StageSrc {
    const __half* x; int ldx;        // rows (plain) / residual stream (rmsnorm) / y (normgate)
    const int* rows;                 // optional row list (shared memory), else rows row0, row0+1, ...
    const __half* nw;                // norm weight
    const __half* z; int ldz;        // gate input of the gated norm
    float eps;
    const float* nw32 = nullptr;     // gated norm only: f32 norm weight (the norm then runs in f32, see stage_finish)
};
struct StageRegs { uint4 a[2], b[2], c[2]; };   // activations, norm weights, gate inputs of the first two units

__device__ __forceinline__ uint4 stage_load(const StageSrc& s, int row0, int col, int k0) {
    int row = s.rows ? s.rows[col] : row0 + col;
    return __ldcg(reinterpret_cast<const uint4*>(s.x + (size_t)row * s.ldx + k0));
}
// norm weights of the warp's first two units: constants, so they may be requested before the
// programmatic-launch wait (they are cold in L2 once per token, a full DRAM round trip)
template <int PRO>
__device__ __forceinline__ void stage_issue_const(StageRegs& sr, const StageSrc& s, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int lgc = 31 - __clz(K >> 8), units = mr << lgc;
    if (PRO == PRO_PLAIN) return;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        int u = warp + j * nw;
        if (u < units) {
            const int k0 = ((u & ((1 << lgc) - 1)) << 8) + lane * 8;
            sr.b[j] = *reinterpret_cast<const uint4*>(s.nw + (pro_is_normgate(PRO) ? (k0 & 127) : k0));
        }
    }
}
template <int PRO>
__device__ __forceinline__ void stage_issue(StageRegs& sr, const StageSrc& s, int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int lgc = 31 - __clz(K >> 8), units = mr << lgc;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        int u = warp + j * nw;
        if (u < units) {
            const int col = u >> lgc, k0 = ((u & ((1 << lgc) - 1)) << 8) + lane * 8;
            sr.a[j] = stage_load(s, row0, col, k0);
            if (pro_is_normgate(PRO)) {
                const int row = s.rows ? s.rows[col] : row0 + col;
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
// Gated RMSNorm of 8 consecutive values of one 128-wide head (the 16 lanes of a half warp hold the head):
// fp16(silu_f32(z) * float(w * fp16(y * inv))); with an f32 weight (PRO_NORMGATE32) the normed value stays
// f32, w * (y * inv) (the reference's promoted variant, SeedlessFusedVerify.swift:766-813).
template <int PRO>
__device__ __forceinline__ uint4 normgate8(uint4 v, uint4 zv, uint4 wv, const float* nw32, int k0, float eps) {
    const __half* yh = reinterpret_cast<const __half*>(&v);
    const __half* zh = reinterpret_cast<const __half*>(&zv);
    const __half* wh = reinterpret_cast<const __half*>(&wv);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { float f = h2f(yh[i]); ss = fmaf(f, f, ss); }
    ss = half_warp_sum(ss);                       // 16 lanes per head of 128
    float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), eps));
    uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float yn = __fmul_rn(h2f(yh[i]), inv);
        float nrm = (PRO == PRO_NORMGATE32) ? __fmul_rn(nw32[(k0 & 127) + i], yn) : h2f(hmul_rn(wh[i], f2h(yn)));
        float zf = h2f(zh[i]);
        oh[i] = f2h(__fmul_rn(__fmul_rn(zf, sigmoid_f(zf)), nrm));
    }
    return o;
}
// RMSNorm: x = w * fp16(h * inv), inv = rsqrt(mean(h^2) + eps) (SeedlessMetalForward.swift:800-827).
// Gated RMSNorm of the GDN out-projection, per head of 128:
// x = fp16(silu_f32(z) * float(w * fp16(y * inv))) (SeedlessFusedVerify.swift:803-813).
// Contains one __syncthreads() for PRO_RMSNORM; the caller synchronises before reading xs.
template <int PRO>
__device__ __forceinline__ void stage_finish(const StageRegs& sr, const XStage& st, const StageSrc& s, int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int lgc = 31 - __clz(K >> 8), chunks = 1 << lgc, units = mr << lgc;
    if (PRO == PRO_RMSNORM) {
        for (int j = 0, u = warp; u < units; ++j, u += nw) {
            const int col = u >> lgc, ch = u & (chunks - 1);
            const uint4 v = (j == 0) ? sr.a[0] : ((j == 1) ? sr.a[1] : stage_load(s, row0, col, (ch << 8) + lane * 8));
            float ss = warp_sum(sumsq8(v));
            if (lane == 0) st.part[col * 16 + ch] = ss;
        }
        __syncthreads();
    }
    for (int j = 0, u = warp; u < units; ++j, u += nw) {
        const int col = u >> lgc, ch = u & (chunks - 1), k0 = (ch << 8) + lane * 8;
        const uint4 v = (j == 0) ? sr.a[0] : ((j == 1) ? sr.a[1] : stage_load(s, row0, col, k0));
        uint4 o;
        if (PRO == PRO_PLAIN) {
            o = v;
        } else if (PRO == PRO_RMSNORM) {
            float tot = 0.f;
            for (int c = 0; c < chunks; ++c) tot += st.part[col * 16 + c];
            float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), s.eps));
            const uint4 wv = (j == 0) ? sr.b[0] : ((j == 1) ? sr.b[1] : *reinterpret_cast<const uint4*>(s.nw + k0));
            o = rms_apply8(v, wv, inv);
        } else {
            const int row = s.rows ? s.rows[col] : row0 + col;
            const uint4 zv = (j == 0) ? sr.c[0] : ((j == 1) ? sr.c[1] : __ldcg(reinterpret_cast<const uint4*>(s.z + (size_t)row * s.ldz + k0)));
            const uint4 wv = (j == 0) ? sr.b[0] : ((j == 1) ? sr.b[1] : *reinterpret_cast<const uint4*>(s.nw + (k0 & 127)));
            o = normgate8<PRO>(v, zv, wv, s.nw32, k0, s.eps);
        }
        store_staged(st, col, k0, o, lane);
    }
}
// whole-prologue forms for kernels that have nothing to overlap with the loads
__device__ __forceinline__ void stage_plain(const XStage& st, const __half* x, int ldx, int row0, int mr, int K) {
    StageSrc s{x, ldx, nullptr, nullptr, nullptr, 0, 0.f};
    StageRegs sr; stage_issue<PRO_PLAIN>(sr, s, row0, mr, K); stage_finish<PRO_PLAIN>(sr, st, s, row0, mr, K);
}
__device__ __forceinline__ void stage_rmsnorm(const XStage& st, const __half* h, int ldh, const __half* w, float eps,
                                              int row0, int mr, int K) {
    StageSrc s{h, ldh, nullptr, w, nullptr, 0, eps};
    StageRegs sr; stage_issue_const<PRO_RMSNORM>(sr, s, mr, K); stage_issue<PRO_RMSNORM>(sr, s, row0, mr, K); stage_finish<PRO_RMSNORM>(sr, st, s, row0, mr, K);
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

// the same fragments from a copy of the unit in shared memory (w: 128 uint4, s: 16 uint4 of the unit)
__device__ __forceinline__ void load_slice_smem(SliceRegs& rg, const uint4* w_unit, const uint4* s_unit, int lane) {
    rg.w[0] = w_unit[lane]; rg.w[1] = w_unit[lane + 32]; rg.w[2] = w_unit[lane + 64]; rg.w[3] = w_unit[lane + 96];
    rg.sc[0] = s_unit[lane >> 2]; rg.sc[1] = s_unit[8 + (lane >> 2)];
}

// (not volatile: pure functions of their operands, so the compiler may interleave independent groups)
__device__ __forceinline__ void mma_f16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// first MMA of a group: the accumulator starts from zero without spending registers on it
__device__ __forceinline__ void mma_f16_z(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// (a & b) | c in one logic instruction (the compiler otherwise spends two when b and c are both constants)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// one word (8 nibbles q0..q7) -> fp16x2 registers {q0,q4}, {q1,q5}, {q2,q6}, {q3,q7}, exact
__device__ __forceinline__ void dequant8(uint32_t w, uint32_t d[4]) {
    const uint32_t w8 = w >> 8;
    const uint32_t mlo = 0x000F000Fu, mhi = 0x00F000F0u, magic = 0x64006400u;
    uint32_t l0 = and_or(w, mlo, magic), h0 = and_or(w, mhi, magic);
    uint32_t l1 = and_or(w8, mlo, magic), h1 = and_or(w8, mhi, magic);
    const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f), k16th = __floats2half2_rn(0.0625f, 0.0625f), k64 = __floats2half2_rn(-64.f, -64.f);
    __half2 r0 = __hsub2(*reinterpret_cast<__half2*>(&l0), k1024);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2*>(&h0), k16th, k64);
    __half2 r2 = __hsub2(*reinterpret_cast<__half2*>(&l1), k1024);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2*>(&h1), k16th, k64);
    d[0] = *reinterpret_cast<uint32_t*>(&r0); d[1] = *reinterpret_cast<uint32_t*>(&r1);
    d[2] = *reinterpret_cast<uint32_t*>(&r2); d[3] = *reinterpret_cast<uint32_t*>(&r3);
}

// B operands of one slice for this lane (MMA column n = lane/4 is pass-row n) and the group sums of
// its two columns: loaded from the activation stage once, reusable for every tile of the same slice
struct XRegs { uint4 x[8]; float2 sx[4]; };
__device__ __forceinline__ void load_xregs(XRegs& xr, const XStage& st, int slice, int n, int t, int mr) {
    const __half* xp = st.xs + (size_t)n * st.stride + slice * 256 + 16 * t;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        xr.x[2 * g] = make_uint4(0, 0, 0, 0); xr.x[2 * g + 1] = make_uint4(0, 0, 0, 0);
        if (n < mr) { xr.x[2 * g] = *reinterpret_cast<const uint4*>(xp + 64 * g); xr.x[2 * g + 1] = *reinterpret_cast<const uint4*>(xp + 64 * g + 8); }
        xr.sx[g] = *reinterpret_cast<const float2*>(st.sxs + (slice * 4 + g) * 8 + 2 * t);
    }
}
// One slice (4 groups) of a 16-row tile.
// accS/accB [4]: (row A, col 2t), (row A, col 2t+1), (row B, col 2t), (row B, col 2t+1).
__device__ __forceinline__ void compute_slice_x(const SliceRegs& r, const XRegs& xr, float accS[4], float accB[4]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint4 X0 = xr.x[2 * g], X1 = xr.x[2 * g + 1];
        const uint4 wv = r.w[g];                      // row A words (x, y), row B words (z, w)
        uint32_t a[4], b[4];
        float c[4];
        dequant8(wv.x, a); dequant8(wv.z, b);
        mma_f16_z(c, a[0], b[0], a[1], b[1], X0.x, X0.y);
        mma_f16(c, a[2], b[2], a[3], b[3], X0.z, X0.w);
        dequant8(wv.y, a); dequant8(wv.w, b);
        mma_f16(c, a[0], b[0], a[1], b[1], X1.x, X1.y);
        mma_f16(c, a[2], b[2], a[3], b[3], X1.z, X1.w);
        const float2 sx2 = xr.sx[g];
        const uint4 sv = r.sc[g >> 1];
        const uint32_t sa_ba = (g & 1) ? sv.z : sv.x, sb_bb = (g & 1) ? sv.w : sv.y;
        float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&sa_ba));    // (scale A, bias A)
        float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&sb_bb));    // (scale B, bias B)
        accS[0] = fmaf(fa.x, c[0], accS[0]); accS[1] = fmaf(fa.x, c[1], accS[1]);
        accS[2] = fmaf(fb.x, c[2], accS[2]); accS[3] = fmaf(fb.x, c[3], accS[3]);
        accB[0] = fmaf(fa.y, sx2.x, accB[0]); accB[1] = fmaf(fa.y, sx2.y, accB[1]);
        accB[2] = fmaf(fb.y, sx2.x, accB[2]); accB[3] = fmaf(fb.y, sx2.y, accB[3]);
    }
}
__device__ __forceinline__ void compute_slice(const SliceRegs& r, const XStage& st, int slice, int n, int t, int mr,
                                              float accS[4], float accB[4]) {
    XRegs xr;
    load_xregs(xr, st, slice, n, t, mr);
    compute_slice_x(r, xr, accS, accB);
}
// scale part + bias part of the slice
__device__ __forceinline__ void finish_acc4(const float accS[4], const float accB[4], int t, float v[4]) {
    (void)t;
    v[0] = accS[0] + accB[0]; v[1] = accS[1] + accB[1]; v[2] = accS[2] + accB[2]; v[3] = accS[3] + accB[3];
}
// value of pass-row j of weight row `row` from the reduced 16x8 tile
__device__ __forceinline__ float tile_value(const float* fin_tile, int row, int j) { return fin_tile[row * 8 + j]; }

// ---- CTA organisation of the split GEMV ----
// A tile is 16 weight rows; its K/256 slices are shared by WPT warps of SPW slices each, and a CTA
// holds TPC tiles.  Every slice's value is kept separate and the slices are summed in ascending
// order whatever the split, so the split is a pure scheduling choice: results do not depend on it.
struct GemvPlan { int upw, tpc, nw, lg_slices; };
// K/256 must be a power of two (K = 256, 512, ... 4096).  A unit is one slice of one tile; a CTA of
// 16 warps takes UPW units per warp (unit u = warp + 16*i -> tile u >> lg_slices, slice u & (slices-1)),
// i.e. TPC = 16*UPW/slices whole tiles.  UPW grows (to at most 3) until `groups` independent
// problems of `ntiles` tiles fit one wave of CTAs (one per multiprocessor).
// nsm: multiprocessors of the device (a wave is one CTA per multiprocessor)
__host__ __device__ inline GemvPlan gemv_plan(int K, int ntiles, int groups, int nsm) {
    GemvPlan p;
    int slices = K >> 8;
    p.lg_slices = 0; while ((1 << p.lg_slices) < slices) ++p.lg_slices;
    p.nw = 16;
    long long units = (long long)ntiles * slices * groups;
    int upw = (int)((units + nsm * 16 - 1) / (nsm * 16));
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

// the same sum taken directly from the partials by the thread that writes the output: value of weight row
// `row` (0..15), pass-row `col` of tile `tl`, slices added in ascending order (identical to reduce_tiles)
__device__ __forceinline__ float tile_sum(const float* red, int tl, int slices, int row, int col) {
    const int j = ((((row & 7) << 2) | (col >> 1)) << 2) | (((row >> 3) << 1) | (col & 1));
    float acc = 0.f;
    for (int sidx = 0; sidx < slices; ++sidx) acc += red[(tl * slices + sidx) * 128 + j];
    return acc;
}

// dynamic shared memory carve-up shared by host (size) and device (pointers)
// Weight stage: the CTA's units (one slice of one tile each: 2048 B of nibbles + 256 B of scales)
// are contiguous in the fragment-major layout, so each round of 16 units arrives by two bulk copies.
struct WStage { uint4* w; uint4* s; uint64_t* bar; };
struct GemvSmem {
    __host__ __device__ static size_t wstage_bytes(int nunits) { return (size_t)nunits * (2048 + 256) + 64; }
    __host__ __device__ static size_t bytes(int rows, int K, int nred, int tpc) {
        size_t xs = (size_t)rows * (K + 8) * 2;
        return xs + (size_t)(K / 64) * 8 * 4 + 8 * 16 * 4 + (size_t)nred * 128 * 4 + (size_t)tpc * 128 * 4 + 128;
    }
    // [weight stage (nunits > 0)] [activation stage] ...; every part stays 16-byte aligned
    __device__ static unsigned char* carve_w(unsigned char* base, int nunits, WStage& ws) {
        ws.w = reinterpret_cast<uint4*>(base);
        ws.s = reinterpret_cast<uint4*>(base + (size_t)nunits * 2048);
        ws.bar = reinterpret_cast<uint64_t*>(base + (size_t)nunits * (2048 + 256));
        return base + wstage_bytes(nunits);
    }
    __device__ static void carve(unsigned char* base, int rows, int K, int nred, int tpc, XStage& st, float*& red, float*& fin, int*& misc) {
        size_t xs = (size_t)rows * (K + 8) * 2;
        st.xs = reinterpret_cast<__half*>(base);
        st.sxs = reinterpret_cast<float*>(base + xs);
        st.part = st.sxs + (K / 64) * 8;
        red = st.part + 8 * 16;
        fin = red + nred * 128;
        misc = reinterpret_cast<int*>(fin + tpc * 128);      // 32 ints
        st.stride = K + 8;
    }
};

// One thread: (init) the mbarriers of a stage, one per round of 16 units; (copy) start the bulk copies of
// the CTA's `nvu` valid units (global unit index u0) and arm each round's barrier for this phase.
// w_all / s_all are the matrix's (or the expert's) arrays.  A stage can be refilled once every
// warp is done reading it; each refill is one more phase of the same barriers.
__device__ __forceinline__ void wstage_init(const WStage& ws, int rounds) {
    for (int i = 0; i < rounds; ++i) mbar_init(ws.bar + i, 1);
    mbar_fence_init();
}
__device__ __forceinline__ void wstage_copy(const WStage& ws, const uint4* w_all, const uint4* s_all, size_t u0, int nvu, int rounds) {
    for (int i = 0; i < rounds; ++i) {
        const int n = min(16, nvu - 16 * i);
        if (n <= 0) break;
        mbar_expect_tx(ws.bar + i, (uint32_t)n * (2048 + 256));
        bulk_g2s(ws.w + (size_t)16 * i * 128, w_all + (u0 + 16 * i) * 128, (uint32_t)n * 2048, ws.bar + i);
        bulk_g2s(ws.s + (size_t)16 * i * 16, s_all + (u0 + 16 * i) * 16, (uint32_t)n * 256, ws.bar + i);
    }
}
__device__ __forceinline__ void wstage_issue(const WStage& ws, const uint4* w_all, const uint4* s_all, size_t u0, int nvu, int rounds) {
    wstage_init(ws, rounds);
    wstage_copy(ws, w_all, s_all, u0, nvu, rounds);
}

}  // namespace sl
