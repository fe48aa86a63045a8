// ep_exchange.cu -- the exchange of expert-parallel batched decode, written over NVLink peer memory.
//
// One process per GPU; rank r owns experts [r*E/R, (r+1)*E/R) and M streams.  Per MoE layer every rank needs the
// normed rows and routing choices of ALL ranks (dispatch), and afterwards gets back, for each of its own (row, k)
// pairs, the one expert output that some rank computed (combine).  Both are tiny (a few hundred KB per layer) and
// latency-bound, so they are done with plain peer stores from this library's own kernels instead of collectives:
//   dispatch  the router kernel's last CTA (k_moe_router, RouterArgs::epd) stores the rank's M normed rows and
//             M*top_k indices straight into every peer's gather buffers, then (after a system fence) a sequence
//             number into that peer's flag word for this rank;
//   wait      k_ep_lists: one CTA waits for all ranks' flags, then groups the pairs that chose a local expert;
//   combine   the down-projection kernel stores each pair's output row directly into the pair OWNER's buffer
//             (ExpertArgs::peer_dbuf); its last CTA raises this rank's flag at every peer, and k_ep_combine waits
//             for all flags before it forms the weighted sum in ascending k.
// Every pair row is written by exactly one rank and arrives unreduced, so the owner sees the bits a single GPU
// computes.  No multicast, no collective inside a step (so a step can be captured in a CUDA graph); every wait is
// bounded and reports through the engine's error word.  There is no counterpart in the reference (one GPU).
#include "kernels.h"

namespace sl {

constexpr long long EP_TIMEOUT = 1ll << 30;        // cycles (~0.5 s) a flag wait may take

// wait until flag >= seq (sequence numbers only grow); false after the budget
__device__ __forceinline__ bool ep_wait_flag(const unsigned* flag, unsigned seq) {
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; ++i) if ((int)(ld_acquire_sys(flag) - seq) >= 0) return true;
        if (clock64() - t0 > EP_TIMEOUT) return false;
    }
}

// One CTA: wait for every rank's dispatch flag, then group the pairs (row, k) whose expert lies in [e0, e1) by
// expert, in the format the expert kernels read.
// dynamic shared memory: npairs ints
__global__ void __launch_bounds__(256) k_ep_lists(EpPeers P, int npairs, int e0, int e1, MoeLists lists, int layer, unsigned* err) {
    extern __shared__ int s_inds[];
    __shared__ int s_cnt[256], s_off[256], s_cur[256];
    const int tid = threadIdx.x;
    if (tid < P.world) { if (!ep_wait_flag(P.flags[P.rank] + tid, ep_seq(P.ctr, layer, 0))) atomicOr(err, 128u); }
    s_cnt[tid] = 0; s_off[tid] = 0; s_cur[tid] = 0;
    __syncthreads();
    const int* inds = P.ibuf[P.rank];
    for (int i = tid; i < npairs; i += 256) { const int ex = __ldcg(inds + i); s_inds[i] = ex; if (ex >= e0 && ex < e1) atomicAdd(&s_cnt[ex], 1); }
    __syncthreads();
    {   // slot numbers and offsets of the local experts by a block scan (thread = expert)
        __shared__ int s_wsum[8], s_wact[8];
        const int warp = tid >> 5, lane = tid & 31;
        const int cnt = (tid >= e0 && tid < e1) ? s_cnt[tid] : 0, act = cnt > 0 ? 1 : 0;
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
        s_off[tid] = off;
        if (act) { lists.slot_expert[slot] = tid; lists.slot_off[slot] = off; lists.slot_cnt[slot] = cnt; }
        if (tid == 255) *lists.n_active = slot + act;
    }
    __syncthreads();
    // (the order of the pairs inside a slot is whatever the atomics give: it only decides which MMA column a row takes)
    for (int i = tid; i < npairs; i += 256) {
        const int ex = s_inds[i];
        if (ex >= e0 && ex < e1) lists.pairs[s_off[ex] + atomicAdd(&s_cur[ex], 1)] = i;
    }
}
void launch_ep_lists(const EpPeers& P, int npairs, int e0, int e1, const MoeLists& lists, int layer, unsigned* err, cudaStream_t st) {
    profile_launch("k_ep_lists", st, [&] { k_ep_lists<<<1, 256, (size_t)npairs * sizeof(int), st>>>(P, npairs, e0, e1, lists, layer, err); return 0; });
}

// grid (M), 256 threads: wait for every rank's combine flag, then
// out/resid[m] (+)= sum_k fp16(d[m*topk + k] * score[m,k]) (ascending k) + sigmoid(sgl[m]) * shared[m]
// (swift/Sources/QwispCore/SeedlessFusedVerify.swift:462-484, SeedlessMetalForward.swift:1024-1028)
__global__ void __launch_bounds__(256) k_ep_combine(EpPeers P, const __half* shared_rows, const __half* scores, const __half* sgl,
                                                    int H, int topk, __half* resid, __half* out, int layer, unsigned* err) {
    const int m = blockIdx.x;
    if ((int)threadIdx.x < P.world) { if (!ep_wait_flag(P.flags[P.rank] + 8 + threadIdx.x, ep_seq(P.ctr, layer, 1))) atomicOr(err, 256u); }
    __syncthreads();
    const __half* dbuf = P.dbuf[P.rank];
    for (int n = threadIdx.x; n < H; n += blockDim.x) {
        __half acc = f2h(0.0f);
        for (int k = 0; k < topk; ++k)
            acc = hadd_rn(acc, hmul_rn(__ldcg(dbuf + (size_t)(m * topk + k) * H + n), scores[m * topk + k]));
        __half res = hadd_rn(acc, hmul_rn(sigmoid_h(sgl[m]), __ldcg(shared_rows + (size_t)m * H + n)));
        if (resid) resid[(size_t)m * H + n] = hadd_rn(resid[(size_t)m * H + n], res);
        else out[(size_t)m * H + n] = res;
    }
}
void launch_ep_combine(const EpPeers& P, const __half* shared_rows, const __half* scores, const __half* sgl, int M, int H, int topk,
                       __half* resid, __half* out, int layer, unsigned* err, cudaStream_t st) {
    profile_launch("k_ep_combine", st, [&] { k_ep_combine<<<M, 256, 0, st>>>(P, shared_rows, scores, sgl, H, topk, resid, out, layer, err); return 0; });
}

__global__ void k_ep_step_end(unsigned* ctr) { *ctr += 1u; }
void launch_ep_step_end(unsigned* ctr, cudaStream_t st) { k_ep_step_end<<<1, 1, 0, st>>>(ctr); count_launch(); }

}  // namespace sl
