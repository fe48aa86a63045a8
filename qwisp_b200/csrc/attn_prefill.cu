// attn_prefill.cu -- causal GQA attention for a prompt chunk (prefill mode): many query rows of ONE stream against the
// paged KV arena, on the tensor cores (mma.sync m16n8k16, fp16 operands, f32 accumulators).
//
// The decode kernel (k_attn_fused) gives every query row its own CTAs and re-reads the keys per row; for a chunk of
// hundreds of rows the keys are the same, so here a CTA owns 64 consecutive rows of one query head and walks the
// keys once, 32 at a time: S = Q K^T (scaled), causal mask by position, online softmax in f32 (running maximum and
// normaliser per row), P rounded to fp16, O += P V.  The epilogue divides by the normaliser, rounds to fp16 and applies
// the sigmoid output gate, like the decode path (swift/Sources/QwispCore/SeedlessMetalForward.swift:4922-4989, :1012-1022).
//
// Prefill-mode numerics: within fp16 tolerance of the decode kernel, not bit-identical to it.  What IS fixed: a row's
// result depends only on its own query and on the keys, which are walked in tiles of 32 aligned to absolute positions;
// a tile that lies entirely behind a row's position leaves that row's state untouched.  So the result does not depend
// on how a prompt is cut into calls or on which rows share a CTA.
//
// Inputs are what k_attn_prep leaves: normed + rotated queries (AttnArgs::qrot) and this call's K / V already in the arena.
#include "kernels.h"
#include "mixer_math.cuh"

namespace sl {

constexpr int AP_BM = 64;            // query rows per CTA (16 per warp)
constexpr int AP_BN = 32;            // keys per tile

__device__ __forceinline__ void ap_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ap_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ap_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ap_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// rows of 256 halves = 32 chunks of 16 bytes; chunk c of row r sits at chunk (c ^ (r & 7)): conflict-free ldmatrix
__device__ __forceinline__ __half* ap_at(__half* base, int row, int chunk) { return base + (size_t)row * ATT_D + ((chunk ^ (row & 7)) << 3); }
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// grid (ceil(M / 64), NH), 128 threads; dynamic shared memory: Q 32 KB + 2 x (K 16 KB + V 16 KB)
__global__ void __launch_bounds__(128) k_attn_prefill(AttnArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __half* Qs = reinterpret_cast<__half*>(smem_raw);                       // [64][256]
    __half* KVs = Qs + AP_BM * ATT_D;                                        // [2][K: 32 x 256 | V: 32 x 256]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * AP_BM, h = blockIdx.y, kvh = h / ATT_G;
    const SegDesc seg = a.segs[0];
    const int slot = seg.slot;
    const int pos0 = a.tab.kv_len[slot];                                     // position of the call's first row
    const int rows = min(AP_BM, a.M - m0);
    const int pos_last = pos0 + m0 + rows - 1;
    const int ntiles = pos_last / AP_BN + 1;
    // ---- the query tile and the first key tile
    for (int i = tid; i < AP_BM * 32; i += 128) {
        const int r = i >> 5, c = i & 31;
        __half* dst = ap_at(Qs, r, c);
        if (r < rows) ap_cp16(dst, a.qrot + ((size_t)(m0 + r) * a.NH + h) * ATT_D + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    auto load_tile = [&](int tile, int buf) {
        __half* Ks = KVs + (size_t)buf * 2 * AP_BN * ATT_D;
        __half* Vs = Ks + AP_BN * ATT_D;
        for (int i = tid; i < AP_BN * 32; i += 128) {
            const int r = i >> 5, c = i & 31;
            const int pos = tile * AP_BN + r;
            if (pos <= pos_last) {
                ap_cp16(ap_at(Ks, r, c), kv_ptr(a, slot, pos, 0, kvh) + c * 8);
                ap_cp16(ap_at(Vs, r, c), kv_ptr(a, slot, pos, 1, kvh) + c * 8);
            } else {                                                         // behind every row of the tile: masked; zero keeps NaN out of P V
                *reinterpret_cast<uint4*>(ap_at(Ks, r, c)) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(ap_at(Vs, r, c)) = make_uint4(0, 0, 0, 0);
            }
        }
        ap_commit();
    };
    load_tile(0, 0);
    // accumulators: this thread's two rows (lane/4 and lane/4 + 8 of the warp's 16), 32 dim tiles of 8
    float o[32][4];
#pragma unroll
    for (int i = 0; i < 32; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }
    float mrun[2] = {-INFINITY, -INFINITY}, lrun[2] = {0.f, 0.f};
    const int prow[2] = {pos0 + m0 + warp * 16 + (lane >> 2), pos0 + m0 + warp * 16 + (lane >> 2) + 8};   // positions of the two rows
    const int pwarp_last = pos0 + m0 + warp * 16 + 15;
    const float scale = 0.0625f;                                             // 256^-0.5
    for (int tile = 0; tile < ntiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < ntiles) { load_tile(tile + 1, buf ^ 1); ap_wait<1>(); } else ap_wait<0>();
        __syncthreads();
        __half* Ks = KVs + (size_t)buf * 2 * AP_BN * ATT_D;
        __half* Vs = Ks + AP_BN * ATT_D;
        if (tile * AP_BN <= pwarp_last) {                                    // else: every key of the tile lies behind all 16 rows
            // ---- S = Q K^T: 4 key groups of 8
            float s[4][4];
#pragma unroll
            for (int n = 0; n < 4; ++n) { s[n][0] = 0.f; s[n][1] = 0.f; s[n][2] = 0.f; s[n][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                uint32_t a0, a1, a2, a3;
                ldsm_x4(a0, a1, a2, a3, ap_at(Qs, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    uint32_t b0, b1, b2, b3;
                    const int mi = lane >> 3;
                    ldsm_x4(b0, b1, b2, b3, ap_at(Ks, (np * 2 + (mi >> 1)) * 8 + (lane & 7), ks * 2 + (mi & 1)));
                    ap_mma(s[np * 2], a0, a1, a2, a3, b0, b1);
                    ap_mma(s[np * 2 + 1], a0, a1, a2, a3, b2, b3);
                }
            }
            // ---- mask, running maximum, P
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = tile * AP_BN + n * 8 + 2 * (lane & 3) + (i & 1);
                    const int rr = i >> 1;
                    const float v = (key <= prow[rr]) ? s[n][i] * scale : -INFINITY;
                    s[n][i] = v;
                    tmax[rr] = fmaxf(tmax[rr], v);
                }
            float alpha[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 1));
                tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 2));
                const float mnew = fmaxf(mrun[rr], tmax[rr]);
                alpha[rr] = (mnew == -INFINITY || mrun[rr] == mnew) ? 1.f : __expf(mrun[rr] - mnew);      // -inf - -inf never evaluated
                mrun[rr] = mnew;
            }
            float psum[2] = {0.f, 0.f};
            uint32_t pa[2][4];                                               // P as A fragments: two key steps of 16
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                float p[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i >> 1;
                    p[i] = (s[n][i] == -INFINITY) ? 0.f : __expf(s[n][i] - mrun[rr]);
                    psum[rr] += p[i];
                }
                pa[n >> 1][(n & 1) * 2] = pack_h2(p[0], p[1]);
                pa[n >> 1][(n & 1) * 2 + 1] = pack_h2(p[2], p[3]);
            }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) lrun[rr] = lrun[rr] * alpha[rr] + psum[rr];
            if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
                for (int i = 0; i < 32; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
            }
            // ---- O += P V
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                for (int dp = 0; dp < 16; ++dp) {                            // pairs of dim tiles
                    uint32_t b0, b1, b2, b3;
                    const int mi = lane >> 3;
                    ldsm_x4_t(b0, b1, b2, b3, ap_at(Vs, kk * 16 + (mi & 1) * 8 + (lane & 7), dp * 2 + (mi >> 1)));
                    ap_mma(o[dp * 2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    ap_mma(o[dp * 2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        }
        __syncthreads();                                                     // the buffer is refilled by the next iteration
    }
    // ---- normalise, round, gate (the row's normaliser is spread over the 4 lanes of a quad)
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        lrun[rr] += __shfl_xor_sync(0xffffffffu, lrun[rr], 1);
        lrun[rr] += __shfl_xor_sync(0xffffffffu, lrun[rr], 2);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = warp * 16 + (lane >> 2) + rr * 8;
        if (r >= rows) continue;
        const int m = m0 + r;
        const __half* gate = a.inproj + (size_t)m * a.ld + (size_t)h * 2 * ATT_D + ATT_D;
        __half* dst = a.gated + ((size_t)m * a.NH + h) * ATT_D;
        const float inv = lrun[rr] == 0.f ? 1.f : 1.f / lrun[rr];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int d = i * 8 + 2 * (lane & 3);
            const __half2 g2 = *reinterpret_cast<const __half2*>(gate + d);
            const __half o0 = hmul_rn(f2h(o[i][rr * 2] * inv), sigmoid_h(__low2half(g2)));
            const __half o1 = hmul_rn(f2h(o[i][rr * 2 + 1] * inv), sigmoid_h(__high2half(g2)));
            *reinterpret_cast<__half2*>(dst + d) = __halves2half2(o0, o1);
        }
    }
}
// Needs: one segment, page_size a multiple of 32, NH = ATT_G * KV.  Returns false when the call is not covered.
bool launch_attn_prefill(const AttnArgs& a, int nsegs, cudaStream_t st) {
    if (nsegs != 1 || a.page_size % AP_BN || a.NH != ATT_G * a.KV || a.row_pos_override) return false;
    const size_t smem = (size_t)(AP_BM * ATT_D + 2 * 2 * AP_BN * ATT_D) * sizeof(__half);
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(k_attn_prefill, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); configured = true; }
    const dim3 grid((unsigned)((a.M + AP_BM - 1) / AP_BM), (unsigned)a.NH);
    profile_launch("k_attn_prefill", st, [&] { k_attn_prefill<<<grid, 128, smem, st>>>(a); return 0; });
    return true;
}

}  // namespace sl
