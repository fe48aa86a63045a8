// synth.cu -- seeded synthetic tensors and the 4-bit affine quantiser, on the device.
//
// The generator is integer-only up to one int->float conversion and two IEEE multiplies, so
// the same (seed, name, index) gives the same bits on any device and on the host:
//   unit(idx) = (sum of eight 16-bit fields of two splitmix64 outputs - 4*65535) * C
// an Irwin-Hall approximation of N(0,1) (support +-4.9 sigma).  The quantiser is the affine
// group-64 4-bit scheme whose dequant contract the reference reads
// (swift/Sources/QwispCore/SeedlessMetalForward.swift:82-87, 219-221): w ~ scale*q + bias.
#include "kernels.h"

namespace sl {

__host__ __device__ static inline uint64_t mix64(uint64_t z) {
    z ^= z >> 30; z *= 0xbf58476d1ce4e5b9ULL;
    z ^= z >> 27; z *= 0x94d049bb133111ebULL;
    z ^= z >> 31; return z;
}
#define SL_GOLD 0x9E3779B97F4A7C15ULL
#define SL_UNIT_C 0x1.3988e2p-16f   /* 1/sqrt(8*(2^32-1)/12) */

uint64_t tensor_seed(uint64_t base_seed, const char* name) {
    uint64_t h = 0xcbf29ce484222325ULL;
    for (const char* p = name; *p; ++p) { h ^= (uint8_t)*p; h *= 0x100000001b3ULL; }
    return mix64(h ^ mix64(base_seed));
}

__device__ __forceinline__ float synth_unit(uint64_t tseed, uint64_t idx) {
    uint64_t r1 = mix64(tseed + SL_GOLD * (2 * idx + 1));
    uint64_t r2 = mix64(r1 ^ 0xD1B54A32D192ED03ULL);
    int32_t s = (int32_t)(r1 & 0xffff) + (int32_t)((r1 >> 16) & 0xffff) + (int32_t)((r1 >> 32) & 0xffff) + (int32_t)(r1 >> 48) +
                (int32_t)(r2 & 0xffff) + (int32_t)((r2 >> 16) & 0xffff) + (int32_t)((r2 >> 32) & 0xffff) + (int32_t)(r2 >> 48);
    s -= 4 * 65535;
    return __fmul_rn((float)s, SL_UNIT_C);
}

__global__ void k_synth_f16(uint64_t tseed, int64_t n, float mean, float std, __half* out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __float2half_rn(__fadd_rn(mean, __fmul_rn(synth_unit(tseed, (uint64_t)i), std)));
}
__global__ void k_synth_f32(uint64_t tseed, int64_t n, float mean, float std, float* out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __fadd_rn(mean, __fmul_rn(synth_unit(tseed, (uint64_t)i), std));
}

// one thread per group of 64 values held in registers as fp16-rounded floats
__device__ __forceinline__ void quantize_group(const float* w, uint32_t* packed8, __half* scale_out, __half* bias_out) {
    float wmin = w[0], wmax = w[0];
#pragma unroll
    for (int j = 1; j < 64; ++j) { wmin = fminf(wmin, w[j]); wmax = fmaxf(wmax, w[j]); }
    const float n_bins = 15.0f, eps = 1e-7f;
    float scale = fmaxf(__fdiv_rn(__fsub_rn(wmax, wmin), n_bins), eps);
    bool side = fabsf(wmin) > fabsf(wmax);
    scale = side ? scale : -scale;
    float edge = side ? wmin : wmax;
    float q0 = roundf(__fdiv_rn(edge, scale));
    bool at_zero = (q0 == 0.0f);
    scale = at_zero ? scale : __fdiv_rn(edge, q0);
    float bias = at_zero ? 0.0f : edge;
    *scale_out = __float2half_rn(scale);
    *bias_out = __float2half_rn(bias);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float q = roundf(__fdiv_rn(__fsub_rn(w[p * 8 + j], bias), scale));
            q = fminf(fmaxf(q, 0.0f), n_bins);
            word |= ((uint32_t)q & 0xfu) << (4 * j);
        }
        packed8[p] = word;
    }
}

__global__ void k_synth_q4(uint64_t tseed, int64_t n_groups, float std, uint32_t* packed, __half* s, __half* b) {
    int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; g < n_groups; g += stride) {
        float w[64];
#pragma unroll
        for (int j = 0; j < 64; ++j)
            w[j] = __half2float(__float2half_rn(__fadd_rn(0.0f, __fmul_rn(synth_unit(tseed, (uint64_t)(g * 64 + j)), std))));
        uint32_t pk[8];
        quantize_group(w, pk, s + g, b + g);
        uint4* dst = reinterpret_cast<uint4*>(packed + g * 8);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    }
}
__global__ void k_quantize_q4(const __half* wsrc, int64_t n_groups, uint32_t* packed, __half* s, __half* b) {
    int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; g < n_groups; g += stride) {
        float w[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) w[j] = __half2float(wsrc[g * 64 + j]);
        uint32_t pk[8];
        quantize_group(w, pk, s + g, b + g);
        uint4* dst = reinterpret_cast<uint4*>(packed + g * 8);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    }
}

static int grid_for(int64_t n, int block) {
    int64_t g = (n + block - 1) / block;
    if (g > 148 * 32) g = 148 * 32;
    if (g < 1) g = 1;
    return (int)g;
}
void launch_synth_f16(uint64_t tseed, int64_t n, float mean, float std, __half* out, cudaStream_t st) {
    k_synth_f16<<<grid_for(n, 256), 256, 0, st>>>(tseed, n, mean, std, out);
}
void launch_synth_f32(uint64_t tseed, int64_t n, float mean, float std, float* out, cudaStream_t st) {
    k_synth_f32<<<grid_for(n, 256), 256, 0, st>>>(tseed, n, mean, std, out);
}
// rows are contiguous groups, so the group index is simply (n*K + k)/64
void launch_synth_q4(uint64_t tseed, int64_t N, int64_t K, float std, uint32_t* packed, __half* s, __half* b, cudaStream_t st) {
    int64_t ng = N * K / 64;
    k_synth_q4<<<grid_for(ng, 128), 128, 0, st>>>(tseed, ng, std, packed, s, b);
}
void launch_quantize_q4(const __half* w, int64_t N, int64_t K, uint32_t* packed, __half* s, __half* b, cudaStream_t st) {
    int64_t ng = N * K / 64;
    k_quantize_q4<<<grid_for(ng, 128), 128, 0, st>>>(w, ng, packed, s, b);
}
// ---- MLX affine layout -> fragment-major layout (see gemv.cuh) ----
__global__ void k_repack_q4(const uint32_t* wA, const __half* sA, const __half* bA, const uint32_t* wB, const __half* sB, const __half* bB,
                            int pair, int64_t tiles, int K, uint4* wr, uint4* sr) {
    const int GP = K / 128, K8 = K / 8, KG = K / 64;
    const int64_t total_w = tiles * GP * 64, total_s = tiles * GP * 8;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < total_w + total_s; i += stride) {
        if (i < total_w) {
            int64_t T = i / (GP * 64); int rem = (int)(i - T * (GP * 64));
            int gp = rem >> 6, gi = (rem >> 5) & 1, lane = rem & 31, r = lane >> 2, t = lane & 3;
            int word = 8 * (2 * gp + gi) + 2 * t;
            int64_t rowA = pair ? 8 * T + r : 16 * T + r, rowB = pair ? 8 * T + r : 16 * T + 8 + r;
            const uint32_t* srcB = pair ? wB : wA;
            wr[i] = make_uint4(wA[rowA * K8 + word], wA[rowA * K8 + word + 1], srcB[rowB * K8 + word], srcB[rowB * K8 + word + 1]);
        } else {
            int64_t j = i - total_w;
            int64_t T = j / (GP * 8); int rem = (int)(j - T * (GP * 8));
            int gp = rem >> 3, r = rem & 7;
            int64_t rowA = pair ? 8 * T + r : 16 * T + r, rowB = pair ? 8 * T + r : 16 * T + 8 + r;
            const __half* sB2 = pair ? sB : sA; const __half* bB2 = pair ? bB : bA;
            __half v[8] = {sA[rowA * KG + 2 * gp], bA[rowA * KG + 2 * gp], sB2[rowB * KG + 2 * gp], bB2[rowB * KG + 2 * gp],
                           sA[rowA * KG + 2 * gp + 1], bA[rowA * KG + 2 * gp + 1], sB2[rowB * KG + 2 * gp + 1], bB2[rowB * KG + 2 * gp + 1]};
            sr[j] = *reinterpret_cast<uint4*>(v);
        }
    }
}
void launch_repack_q4(const Q4W& a, const Q4W* b_pair, uint4* wr, uint4* sr, cudaStream_t st) {
    int64_t tiles = b_pair ? a.N / 8 : a.N / 16;
    int64_t total = tiles * (a.K / 128) * 72;
    k_repack_q4<<<grid_for(total, 256), 256, 0, st>>>(a.w, a.s, a.b, b_pair ? b_pair->w : nullptr, b_pair ? b_pair->s : nullptr,
                                                       b_pair ? b_pair->b : nullptr, b_pair ? 1 : 0, tiles, a.K, wr, sr);
}
void host_synth_tokens(uint64_t tseed, int64_t n, int32_t vocab, int32_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = (int32_t)(mix64(tseed + SL_GOLD * (2 * (uint64_t)i + 1)) % (uint64_t)vocab);
}

}  // namespace sl
