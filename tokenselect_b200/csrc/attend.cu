// Sparse paged decode attention over the selected pool rows, split over the list with a
// log-sum-exp merge.
//
// Replaces the third-party paged decode call at token_retrieval.py:815-825 (planned at :802-813):
// page size 1, query rotated at position count-1, the j-th listed key at position j (rotate-half
// pairing, frequencies / rope_scale), logits * sm_scale, optional soft cap, fp32 softmax, values
// un-rotated, KV head = h / group.
//
// Split kernel: grid (chunks, batch), 8 warps.  A warp owns one KV head (and, when fewer than 8 KV
// heads are local, one residue class of the chunk's tokens); lane l holds elements
// [P*l, P*l+P) and [D/2 + P*l, D/2 + P*l + P) of a row, i.e. both members of each rotation pair, so
// the rotation needs no exchange; dot products are finished with warp shuffles.  All K/V rows of the
// warp's tokens are requested before the first is used.
#include "common.cuh"

namespace ts {

constexpr int kAttnWarps = kAttnThreads / 32;

template <typename T, int P> struct RowFrag;           // the lane's 2*P elements of one row
template <int P> struct RowFrag<__nv_bfloat16, P> {
    uint32_t lo, hi;                                   // P bf16 values each, element 0 in the low half
    __device__ __forceinline__ void load(const __nv_bfloat16* row, int lane, int half) {
        if (P == 2) {
            lo = *reinterpret_cast<const uint32_t*>(row + 2 * lane);
            hi = *reinterpret_cast<const uint32_t*>(row + half + 2 * lane);
        } else {
            lo = *reinterpret_cast<const unsigned short*>(row + lane);
            hi = *reinterpret_cast<const unsigned short*>(row + half + lane);
        }
    }
    __device__ __forceinline__ float l(int e) const { return __uint_as_float(e == 0 ? (lo << 16) : (lo & 0xFFFF0000u)); }
    __device__ __forceinline__ float h(int e) const { return __uint_as_float(e == 0 ? (hi << 16) : (hi & 0xFFFF0000u)); }
};
template <int P> struct RowFrag<float, P> {
    float lo[P], hi[P];
    __device__ __forceinline__ void load(const float* row, int lane, int half) {
        if (P == 2) {
            const float2 a = *reinterpret_cast<const float2*>(row + 2 * lane);
            const float2 c = *reinterpret_cast<const float2*>(row + half + 2 * lane);
            lo[0] = a.x; lo[P - 1] = a.y; hi[0] = c.x; hi[P - 1] = c.y;
        } else {
            lo[0] = row[lane];
            hi[0] = row[half + lane];
        }
    }
    __device__ __forceinline__ float l(int e) const { return lo[e]; }
    __device__ __forceinline__ float h(int e) const { return hi[e]; }
};

template <typename T, int P, int GMAX>
__global__ void __launch_bounds__(kAttnThreads) attend_split_kernel(const LayerParams p) {
    constexpr int D = 64 * P, HALF = 32 * P;
    constexpr int UNROLL = sizeof(T) == 2 ? 8 : 4;
    __shared__ float sm_o[kAttnWarps][GMAX][D];
    __shared__ float2 sm_ml[kAttnWarps][GMAX];
    if (*(volatile int*)p.err != 0) return;

    const int b = blockIdx.y, chunk = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int count = p.sel_count[b];
    const int CH = p.attn_chunk_tokens;
    const int base = chunk * CH;
    if (base >= count) return;
    const int cnt = min(CH, count - base);
    const int hkv = p.hkv, G = p.group, hq = p.hq;
    const int nsub = hkv >= kAttnWarps ? 1 : kAttnWarps / hkv;
    const int* slots = p.sel_slots + (size_t)b * p.n_sel + base;
    const T* kpool = reinterpret_cast<const T*>(p.k_pool);
    const T* vpool = reinterpret_cast<const T*>(p.v_pool);
    const T* q = reinterpret_cast<const T*>(p.q) + (size_t)b * hq * D;
    const float2* cs_q = p.attn_cs + (size_t)(count - 1) * HALF + P * lane;

    for (int unit = warp; unit < hkv * nsub; unit += kAttnWarps) {
        const int kv = unit % hkv, sub = unit / hkv;
        // query heads of this KV head, rotated at position count-1
        float q1[GMAX][P], q2[GMAX][P];
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            RowFrag<T, P> f;
            if (g < G) f.load(q + (size_t)(kv * G + g) * D, lane, HALF);
#pragma unroll
            for (int e = 0; e < P; ++e) {
                float x1 = g < G ? f.l(e) : 0.f, x2 = g < G ? f.h(e) : 0.f;
                float2 cs = cs_q[e];
                q1[g][e] = x1 * cs.x - x2 * cs.y;
                q2[g][e] = x2 * cs.x + x1 * cs.y;
            }
        }
        float m[GMAX], l[GMAX], o1[GMAX][P], o2[GMAX][P];
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
            for (int e = 0; e < P; ++e) { o1[g][e] = 0.f; o2[g][e] = 0.f; }
        }
        // tokens of this unit: j = sub, sub + nsub, ... < cnt
        for (int j0 = sub; j0 < cnt; j0 += nsub * UNROLL) {
            RowFrag<T, P> kf[UNROLL], vf[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int j = j0 + u * nsub;
                if (j < cnt) {
                    const size_t r = ((size_t)__ldg(slots + j) * hkv + kv) * D;
                    kf[u].load(kpool + r, lane, HALF);
                    vf[u].load(vpool + r, lane, HALF);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int j = j0 + u * nsub;
                if (j >= cnt) break;
                const float2* cs_k = p.attn_cs + (size_t)(base + j) * HALF + P * lane;
                float kr1[P], kr2[P];
#pragma unroll
                for (int e = 0; e < P; ++e) {
                    float2 cs = cs_k[e];
                    float x1 = kf[u].l(e), x2 = kf[u].h(e);
                    kr1[e] = x1 * cs.x - x2 * cs.y;
                    kr2[e] = x2 * cs.x + x1 * cs.y;
                }
                float s[GMAX];
#pragma unroll
                for (int g = 0; g < GMAX; ++g) {
                    float a = 0.f;
#pragma unroll
                    for (int e = 0; e < P; ++e) a += q1[g][e] * kr1[e] + q2[g][e] * kr2[e];
                    s[g] = a;
                }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
#pragma unroll
                    for (int g = 0; g < GMAX; ++g)
                        if (g < G) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
                }
#pragma unroll
                for (int g = 0; g < GMAX; ++g) {
                    if (g < G) {
                        float x = s[g] * p.sm_scale;
                        if (p.logit_cap > 0.f) x = p.logit_cap * tanhf(x / p.logit_cap);
                        const float mn = fmaxf(m[g], x);
                        const float sc = expf(m[g] - mn);
                        const float pe = expf(x - mn);
                        l[g] = l[g] * sc + pe;
                        m[g] = mn;
#pragma unroll
                        for (int e = 0; e < P; ++e) {
                            o1[g][e] = o1[g][e] * sc + pe * vf[u].l(e);
                            o2[g][e] = o2[g][e] * sc + pe * vf[u].h(e);
                        }
                    }
                }
            }
        }
        // partial of this warp -> shared memory
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            if (g < G) {
#pragma unroll
                for (int e = 0; e < P; ++e) {
                    sm_o[warp][g][P * lane + e] = o1[g][e];
                    sm_o[warp][g][HALF + P * lane + e] = o2[g][e];
                }
                if (lane == 0) sm_ml[warp][g] = make_float2(m[g], l[g]);
            }
        }
        if (hkv * nsub > kAttnWarps) {
            // more units than warps (hkv > 8): write this unit straight out, no cross-warp merge
            __syncwarp();
            for (int g = 0; g < G; ++g) {
                const int h = kv * G + g;
                float* dst = p.attn_o + (((size_t)b * p.attn_chunks + chunk) * hq + h) * D;
                for (int e = lane; e < D; e += 32) dst[e] = sm_o[warp][g][e];
                if (lane == 0) p.attn_ml[((size_t)b * p.attn_chunks + chunk) * hq + h] = sm_ml[warp][g];
            }
            __syncwarp();
        }
    }
    if (hkv * nsub > kAttnWarps) return;
    __syncthreads();
    // merge the nsub warps of each KV head and write the chunk's partial
    for (int idx = threadIdx.x; idx < hq * D; idx += kAttnThreads) {
        const int h = idx / D, e = idx - h * D;
        const int kv = h / G, g = h - kv * G;
        float mm = -INFINITY;
        for (int s = 0; s < nsub; ++s) mm = fmaxf(mm, sm_ml[kv + s * hkv][g].x);
        float acc = 0.f, ll = 0.f;
        for (int s = 0; s < nsub; ++s) {
            const float2 ml = sm_ml[kv + s * hkv][g];
            const float w = (ml.x == -INFINITY) ? 0.f : expf(ml.x - mm);
            acc += sm_o[kv + s * hkv][g][e] * w;
            ll += ml.y * w;
        }
        p.attn_o[(((size_t)b * p.attn_chunks + chunk) * hq + h) * D + e] = acc;
        if (e == 0) p.attn_ml[((size_t)b * p.attn_chunks + chunk) * hq + h] = make_float2(mm, ll);
    }
}

// grid = (hq, batch), block = D.
template <typename T>
__global__ void attend_merge_kernel(const LayerParams p) {
    if (*(volatile int*)p.err != 0) return;
    const int h = blockIdx.x, b = blockIdx.y, e = threadIdx.x;
    const int D = p.d, hq = p.hq;
    const int count = p.sel_count[b];
    const int chunks = (count + p.attn_chunk_tokens - 1) / p.attn_chunk_tokens;
    const float2* ml = p.attn_ml + (size_t)b * p.attn_chunks * hq + h;
    const float* o = p.attn_o + ((size_t)b * p.attn_chunks * hq + h) * D + e;
    float mm = -INFINITY;
    for (int c = 0; c < chunks; ++c) mm = fmaxf(mm, ml[(size_t)c * hq].x);
    float acc = 0.f, ll = 0.f;
    for (int c = 0; c < chunks; ++c) {
        const float2 v = ml[(size_t)c * hq];
        const float w = (v.x == -INFINITY) ? 0.f : expf(v.x - mm);
        acc += o[(size_t)c * hq * D] * w;
        ll += v.y * w;
    }
    reinterpret_cast<T*>(p.out)[((size_t)b * hq + h) * D + e] = from_f32<T>(acc / ll);
}

template <typename T, int P>
static cudaError_t launch_attend_t(const LayerParams& p, const Launch& l) {
    dim3 grid(p.attn_chunks, p.batch);
    stage_begin(l, kStageAttendSplit);
    if (p.group <= 4) attend_split_kernel<T, P, 4><<<grid, kAttnThreads, 0, l.stream>>>(p);
    else attend_split_kernel<T, P, 8><<<grid, kAttnThreads, 0, l.stream>>>(p);
    stage_end(l);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    stage_begin(l, kStageAttendMerge);
    attend_merge_kernel<T><<<dim3(p.hq, p.batch), p.d, 0, l.stream>>>(p);
    stage_end(l);
    return cudaGetLastError();
}

cudaError_t launch_attend(const LayerParams& p, const Launch& l) {
    if (l.dtype == TS_DTYPE_BF16) {
        if (p.d == 128) return launch_attend_t<__nv_bfloat16, 2>(p, l);
        return launch_attend_t<__nv_bfloat16, 1>(p, l);
    }
    if (p.d == 128) return launch_attend_t<float, 2>(p, l);
    return launch_attend_t<float, 1>(p, l);
}

}  // namespace ts
