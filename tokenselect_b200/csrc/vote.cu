// Soft vote: second half of the per-head softmax and the head sum,
//
//   vote[t] = sum_c exp(logit[c, t] - M_c) / L_c ,   (M_c, L_c) = softmax statistics of head c,
//
// i.e. torch.softmax(scores, dim=-1).sum(dim=0) (token_retrieval.py:361) in fp32, plus the optional
// sliding max over votes (:366-369) and the first-level histogram of the radix top-k (:371).
#include "common.cuh"

namespace ts {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ unsigned vote_bin(float v) {
    // votes are >= 0, so the raw bit pattern orders like the value; bits [30:20] index the bin
    return (__float_as_uint(v) >> 20) & (kHistBins - 1);
}

// grid = (gx, batch), block = 256.
template <bool kWithHist>
__global__ void __launch_bounds__(256) vote_kernel(const LayerParams p) {
    __shared__ Plan plan;
    __shared__ float s_m[kMaxHq], s_inv[kMaxHq];
    __shared__ unsigned s_hist[kWithHist ? kHistBins : 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (!build_plan(p, plan)) return;
    const int b = blockIdx.y;
    if (plan.flag[b] != TS_FLAG_RECOMPUTE) return;
    const int nc = plan.nc[b], hq = p.hq;

    // merge the scoring CTAs' (max, sum exp) partials of this request: one warp per head
    for (int c = warp; c < hq; c += 8) {
        float m = -INFINITY, l = 0.f;
        for (int i = lane; i < p.score_grid; i += 32) {
            float2 v = p.partials[((size_t)b * p.score_grid + i) * hq + c];
            ml_merge(m, l, v.x, v.y);
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            float mo = __shfl_xor_sync(0xffffffffu, m, o);
            float lo = __shfl_xor_sync(0xffffffffu, l, o);
            ml_merge(m, l, mo, lo);
        }
        if (lane == 0) { s_m[c] = m; s_inv[c] = 1.f / l; }
    }
    if (kWithHist)
        for (int i = tid; i < kHistBins; i += 256) s_hist[i] = 0u;
    __syncthreads();

    const float* lg = p.logits + (size_t)plan.off[b] * hq;
    float* votes = p.votes + plan.off[b];
    for (int t = blockIdx.x * 256 + tid; t < nc; t += gridDim.x * 256) {
        const float* row = lg + (size_t)t * hq;
        float v = 0.f;
        if ((hq & 3) == 0) {
            for (int c = 0; c < hq; c += 4) {
                float4 x = *reinterpret_cast<const float4*>(row + c);
                v += exp2f((x.x - s_m[c]) * kLog2e) * s_inv[c];
                v += exp2f((x.y - s_m[c + 1]) * kLog2e) * s_inv[c + 1];
                v += exp2f((x.z - s_m[c + 2]) * kLog2e) * s_inv[c + 2];
                v += exp2f((x.w - s_m[c + 3]) * kLog2e) * s_inv[c + 3];
            }
        } else {
            for (int c = 0; c < hq; ++c) v += exp2f((row[c] - s_m[c]) * kLog2e) * s_inv[c];
        }
        votes[t] = v;
        if (kWithHist) atomicAdd(&s_hist[vote_bin(v)], 1u);
    }
    if (kWithHist) {
        __syncthreads();
        unsigned* gh = p.hist + (size_t)b * kHistBins;
        for (int i = tid; i < kHistBins; i += 256) {
            unsigned c = s_hist[i];
            if (c) atomicAdd(gh + i, c);
        }
    }
}

// Optional max-pool (window K, padding (K-1)/2, stride 1, implicit -inf padding) followed by the
// histogram.  Used when the votes change after vote_kernel: pooling on, or a tensor-parallel sum.
// grid = (gx, batch), block = 256.
__global__ void __launch_bounds__(256) pool_hist_kernel(const LayerParams p) {
    __shared__ Plan plan;
    __shared__ unsigned s_hist[kHistBins];
    const int tid = threadIdx.x;
    if (!build_plan(p, plan)) return;
    const int b = blockIdx.y;
    if (plan.flag[b] != TS_FLAG_RECOMPUTE) return;
    const int nc = plan.nc[b];
    const int K = p.kernel_size;
    const int ne = pooled_len(nc, K);
    const int pad = K > 0 ? (K - 1) / 2 : 0;
    for (int i = tid; i < kHistBins; i += 256) s_hist[i] = 0u;
    __syncthreads();
    const float* src = p.votes + plan.off[b];
    float* dst = p.votes_pool + plan.off[b];
    for (int t = blockIdx.x * 256 + tid; t < ne; t += gridDim.x * 256) {
        float v;
        if (K > 0) {
            int lo = max(t - pad, 0), hi = min(t - pad + K - 1, nc - 1);
            v = src[lo];
            for (int j = lo + 1; j <= hi; ++j) v = fmaxf(v, src[j]);
            dst[t] = v;
        } else {
            v = src[t];
        }
        atomicAdd(&s_hist[vote_bin(v)], 1u);
    }
    __syncthreads();
    unsigned* gh = p.hist + (size_t)b * kHistBins;
    for (int i = tid; i < kHistBins; i += 256) {
        unsigned c = s_hist[i];
        if (c) atomicAdd(gh + i, c);
    }
}

static int vote_gx(const LayerParams& p, const Launch& l) {
    int gx = (2 * l.num_sms) / (p.batch > 0 ? p.batch : 1);
    return gx < 1 ? 1 : gx;
}

cudaError_t launch_vote(const LayerParams& p, const Launch& l, bool with_hist) {
    dim3 grid(vote_gx(p, l), p.batch), block(256);
    if (with_hist) vote_kernel<true><<<grid, block, 0, l.stream>>>(p);
    else vote_kernel<false><<<grid, block, 0, l.stream>>>(p);
    ++*l.launch_count;
    return cudaGetLastError();
}

cudaError_t launch_pool_hist(const LayerParams& p, const Launch& l) {
    dim3 grid(vote_gx(p, l), p.batch), block(256);
    pool_hist_kernel<<<grid, block, 0, l.stream>>>(p);
    ++*l.launch_count;
    return cudaGetLastError();
}

}  // namespace ts
