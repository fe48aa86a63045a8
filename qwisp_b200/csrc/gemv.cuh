// gemv.cuh -- 4-bit group-64 GEMV family ("F1": decode / verify rows, M-invariant per row).
//
// y[m, n] = sum_k x[m, k] * (scale[n, k/64] * q[n, k] + bias[n, k/64]),  q = nibble k%8 of
// word w[n, k/8] (low nibble first) -- the MLX affine layout of the reference
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:219-221, 238-310).
//
// B200 formulation.  HBM-bound, so the goal is few instructions per weight nibble:
//   * a warp owns 16 weight rows x 256 inputs (one "slice" = 4 groups); thread (r = lane/4,
//     t = lane%4) loads 8 bytes per row and group for rows r and r+8 -- 16 k values of group g;
//   * nibbles become fp16 tensor-core operands with ONE and-mask each: (w & 0x000f000f) read
//     as two fp16 subnormals is (q0, q4) * 2^-24, (w & 0x00f000f0) is (q1, q5) * 2^-20; the
//     activations are staged in shared memory in the matching order with the odd ones
//     pre-divided by 16 (the same 16^j trick MLX's qmv uses, SeedlessMetalForward.swift:238-258);
//   * mma.sync m16n8k16 accumulates sum q*x in fp32 per group (products are exact), then
//     acc += scale * C + bias * sum(x): two FMAs per group and output instead of per element;
//   * the 8 MMA columns are 8 activation rows, so M <= 8 rows share one pass over the weights
//     and each row's result is independent of M (columns of an MMA do not interact);
//   * slices of one 16-row tile are reduced across warps through shared memory in slice order.
// If a device's tensor cores flushed fp16 subnormals, the EXACT variant converts the nibbles
// to integer-valued fp16 first (one extra HSUB2 per pair); the engine picks by a self-test.
#pragma once
#include "common.cuh"

namespace sl {

enum { PRO_PLAIN = 0, PRO_RMSNORM = 1, PRO_NORMGATE = 2 };
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_ARGMAX = 3 };

struct XStage {
    __half* xs;      // [rows][K+8] permuted / pre-scaled activations
    float* sxs;      // [K/64][8] per-group sums of x
    float* part;     // [8][16] scratch for the rmsnorm prologue
    int stride;      // K + 8 (halfs)
};

// (x0..x7) -> (x0,x4, x1/16,x5/16, x2,x6, x3/16,x7/16)
__device__ __forceinline__ uint4 permute_scale8(uint4 v) {
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    uint32_t p1 = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    uint32_t p3 = __byte_perm(v.y, v.w, 0x7632);
    const __half2 sc = __floats2half2_rn(0.0625f, 0.0625f);
    __half2 q1 = __hmul2(*reinterpret_cast<__half2*>(&p1), sc);
    __half2 q3 = __hmul2(*reinterpret_cast<__half2*>(&p3), sc);
    o.y = *reinterpret_cast<uint32_t*>(&q1);
    o.w = *reinterpret_cast<uint32_t*>(&q3);
    return o;
}
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
// lane holds 8 consecutive activations of column `col` starting at k0 (multiple of 8): write
// them staged and accumulate the group sum (8 consecutive lanes cover one group of 64)
__device__ __forceinline__ void store_staged(const XStage& st, int col, int k0, uint4 v, int lane) {
    float s = sum8_f32(v);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 7) == 0) st.sxs[(k0 >> 6) * 8 + col] = s;
    *reinterpret_cast<uint4*>(st.xs + (size_t)col * st.stride + k0) = permute_scale8(v);
}

// ---- prologues: stage `mr` activation rows (first global row = row0) of width K ----
// plain rows x[row*ldx + k]
__device__ __forceinline__ void stage_plain(const XStage& st, const __half* x, int ldx, int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8;
    for (int u = warp; u < mr * chunks; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;
        uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)(row0 + col) * ldx + k0);
        store_staged(st, col, k0, v, lane);
    }
}
// rows gathered through an index list: row of column c = rows[c]
__device__ __forceinline__ void stage_gather(const XStage& st, const __half* x, int ldx, const int* rows, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8;
    for (int u = warp; u < mr * chunks; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;
        uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)rows[col] * ldx + k0);
        store_staged(st, col, k0, v, lane);
    }
}
// RMSNorm prologue: x = w * fp16(h * inv), inv = rsqrt(mean(h^2) + eps)
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:800-827).  K <= 4096.
__device__ __forceinline__ void stage_rmsnorm(const XStage& st, const __half* h, int ldh, const __half* w, float eps,
                                              int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8;
    for (int u = warp; u < mr * chunks; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;
        uint4 v = *reinterpret_cast<const uint4*>(h + (size_t)(row0 + col) * ldh + k0);
        const __half2* hh = reinterpret_cast<const __half2*>(&v);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __half22float2(hh[i]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
        ss = warp_sum(ss);
        if (lane == 0) st.part[col * 16 + ch] = ss;
    }
    __syncthreads();
    for (int u = warp; u < mr * chunks; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;
        float tot = 0.f;
        for (int c = 0; c < chunks; ++c) tot += st.part[col * 16 + c];
        float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), eps));
        uint4 v = *reinterpret_cast<const uint4*>(h + (size_t)(row0 + col) * ldh + k0);
        uint4 wv = *reinterpret_cast<const uint4*>(w + k0);
        const __half* hv = reinterpret_cast<const __half*>(&v);
        const __half* wh = reinterpret_cast<const __half*>(&wv);
        uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) oh[i] = hmul_rn(wh[i], f2h(__fmul_rn(h2f(hv[i]), inv)));
        store_staged(st, col, k0, o, lane);
    }
}
// gated RMSNorm prologue of the GDN out-projection: per head of 128,
// x = fp16(silu_f32(z) * float(w * fp16(y * inv)))  (SeedlessFusedVerify.swift:803-813)
__device__ __forceinline__ void stage_normgate(const XStage& st, const __half* y, int ldy, const __half* z, int ldz,
                                               const __half* w, float eps, int row0, int mr, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int chunks = K >> 8;
    for (int u = warp; u < mr * chunks; u += nw) {
        int col = u / chunks, ch = u - col * chunks;
        int k0 = ch * 256 + lane * 8;                       // 16 lanes per head of 128
        uint4 v = *reinterpret_cast<const uint4*>(y + (size_t)(row0 + col) * ldy + k0);
        uint4 zv = *reinterpret_cast<const uint4*>(z + (size_t)(row0 + col) * ldz + k0);
        uint4 wv = *reinterpret_cast<const uint4*>(w + (k0 & 127));
        const __half* yh = reinterpret_cast<const __half*>(&v);
        const __half* zh = reinterpret_cast<const __half*>(&zv);
        const __half* wh = reinterpret_cast<const __half*>(&wv);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { float f = h2f(yh[i]); ss = fmaf(f, f, ss); }
        ss = half_warp_sum(ss);
        float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), eps));
        uint4 o; __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float nrm = h2f(hmul_rn(wh[i], f2h(__fmul_rn(h2f(yh[i]), inv))));
            float zf = h2f(zh[i]);
            oh[i] = f2h(__fmul_rn(__fmul_rn(zf, sigmoid_f(zf)), nrm));
        }
        store_staged(st, col, k0, o, lane);
    }
}

// ---- weight slice held in registers: rows A and B of this lane, 4 groups (256 inputs) ----
struct SliceRegs { uint2 wA[4], wB[4]; uint2 sA, bA, sB, bB; };

// wA/wB: row starts (uint32 words); sA..bB: row starts of the fp16 scale / bias arrays
__device__ __forceinline__ void load_slice(SliceRegs& r, const uint32_t* wA, const uint32_t* wB, const __half* sA,
                                           const __half* bA, const __half* sB, const __half* bB, int slice, int t) {
    const int w0 = slice * 32 + 2 * t;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        r.wA[g] = ldg_nc_u2(wA + w0 + 8 * g);
        r.wB[g] = ldg_nc_u2(wB + w0 + 8 * g);
    }
    r.sA = ldg_nc_u2(sA + slice * 4); r.bA = ldg_nc_u2(bA + slice * 4);
    r.sB = ldg_nc_u2(sB + slice * 4); r.bB = ldg_nc_u2(bB + slice * 4);
}

template <bool EXACT>
__device__ __forceinline__ uint32_t nib(uint32_t m) {
    if (EXACT) {
        uint32_t v = m | 0x64006400u;                          // 1024 + q (or 1024 + 16 q)
        const __half2 off = __floats2half2_rn(1024.f, 1024.f);
        __half2 r = __hsub2(*reinterpret_cast<__half2*>(&v), off);
        return *reinterpret_cast<uint32_t*>(&r);
    }
    return m;                                                   // subnormal fp16: q * 2^-24 (or q * 2^-20)
}

// accS/accB [4]: (row A, col 2t), (row A, col 2t+1), (row B, col 2t), (row B, col 2t+1)
template <bool EXACT>
__device__ __forceinline__ void compute_slice(const SliceRegs& r, const XStage& st, int slice, int n, int t, bool col_active,
                                              float accS[4], float accB[4]) {
    const __half* xp = st.xs + (size_t)n * st.stride + slice * 256 + 16 * t;
    const __half* sAh = reinterpret_cast<const __half*>(&r.sA);
    const __half* bAh = reinterpret_cast<const __half*>(&r.bA);
    const __half* sBh = reinterpret_cast<const __half*>(&r.sB);
    const __half* bBh = reinterpret_cast<const __half*>(&r.bB);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 X0 = make_uint4(0, 0, 0, 0), X1 = make_uint4(0, 0, 0, 0);
        if (col_active) {
            X0 = *reinterpret_cast<const uint4*>(xp + 64 * g);
            X1 = *reinterpret_cast<const uint4*>(xp + 64 * g + 8);
        }
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        {
            uint32_t ua = r.wA[g].x, ub = r.wB[g].x, va = ua >> 8, vb = ub >> 8;
            mma16816(c, nib<EXACT>(ua & 0x000f000fu), nib<EXACT>(ub & 0x000f000fu), nib<EXACT>(ua & 0x00f000f0u), nib<EXACT>(ub & 0x00f000f0u), X0.x, X0.y);
            mma16816(c, nib<EXACT>(va & 0x000f000fu), nib<EXACT>(vb & 0x000f000fu), nib<EXACT>(va & 0x00f000f0u), nib<EXACT>(vb & 0x00f000f0u), X0.z, X0.w);
        }
        {
            uint32_t ua = r.wA[g].y, ub = r.wB[g].y, va = ua >> 8, vb = ub >> 8;
            mma16816(c, nib<EXACT>(ua & 0x000f000fu), nib<EXACT>(ub & 0x000f000fu), nib<EXACT>(ua & 0x00f000f0u), nib<EXACT>(ub & 0x00f000f0u), X1.x, X1.y);
            mma16816(c, nib<EXACT>(va & 0x000f000fu), nib<EXACT>(vb & 0x000f000fu), nib<EXACT>(va & 0x00f000f0u), nib<EXACT>(vb & 0x00f000f0u), X1.z, X1.w);
        }
        float2 sx = *reinterpret_cast<const float2*>(st.sxs + (slice * 4 + g) * 8 + 2 * t);
        float sa = h2f(sAh[g]), ba = h2f(bAh[g]), sb = h2f(sBh[g]), bb = h2f(bBh[g]);
        accS[0] = fmaf(sa, c[0], accS[0]); accS[1] = fmaf(sa, c[1], accS[1]);
        accS[2] = fmaf(sb, c[2], accS[2]); accS[3] = fmaf(sb, c[3], accS[3]);
        accB[0] = fmaf(ba, sx.x, accB[0]); accB[1] = fmaf(ba, sx.y, accB[1]);
        accB[2] = fmaf(bb, sx.x, accB[2]); accB[3] = fmaf(bb, sx.y, accB[3]);
    }
}
template <bool EXACT>
__device__ __forceinline__ float finish_acc(float s, float b) { return EXACT ? (s + b) : fmaf(s, 16777216.0f, b); }

// cross-warp reduction of a 16x8 tile in slice order: red [nw][128] -> fin[row*8 + col], where
// element i of a warp's 128 is lane = i>>2, ci = i&3, row = (lane>>2) + 8*(ci>>1), col = 2*(lane&3) + (ci&1).
// Contains two __syncthreads().
__device__ __forceinline__ void reduce_tile(float* red, float* fin, const float v[4], int nw) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    *reinterpret_cast<float4*>(red + warp * 128 + lane * 4) = make_float4(v[0], v[1], v[2], v[3]);
    __syncthreads();
    for (int i = threadIdx.x; i < 128; i += blockDim.x) {
        float acc = 0.f;
        for (int w = 0; w < nw; ++w) acc += red[w * 128 + i];
        int l = i >> 2, ci = i & 3;
        int row = (l >> 2) + 8 * (ci >> 1), col = 2 * (l & 3) + (ci & 1);
        fin[row * 8 + col] = acc;
    }
    __syncthreads();
}

// dynamic shared memory carve-up shared by host (size) and device (pointers)
struct GemvSmem {
    __host__ __device__ static size_t bytes(int rows, int K, int nw) {
        size_t xs = ((size_t)rows * (K + 8) * 2 + 15) & ~(size_t)15;
        return xs + (size_t)(K / 64) * 8 * 4 + 8 * 16 * 4 + (size_t)nw * 128 * 4 + 128 * 4 + 64;
    }
    __device__ static void carve(unsigned char* base, int rows, int K, int nw, XStage& st, float*& red, float*& fin, int*& misc) {
        size_t xs = ((size_t)rows * (K + 8) * 2 + 15) & ~(size_t)15;
        st.xs = reinterpret_cast<__half*>(base);
        st.sxs = reinterpret_cast<float*>(base + xs);
        st.part = st.sxs + (K / 64) * 8;
        red = st.part + 8 * 16;
        fin = red + nw * 128;
        misc = reinterpret_cast<int*>(fin + 128);
        st.stride = K + 8;
    }
};

}  // namespace sl
