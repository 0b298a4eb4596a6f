// Per-request preparation of one layer step, as device functions shared by the stand-alone
// prepare kernel (tensor-parallel form) and phase 0 of the fused selection kernel:
// K/V append, scoring-query rotation, cosine terms of the selection cache and the
// recompute / reuse / dense decision.
//
// Replaces store_kv_cache (token_retrieval.py:844-854), the query rotation at :380-388 with
// RotaryEmbedding.apply_rotary_pos_emb (:98-107), the guard at :376-378 and the (intended)
// selection-cache rule at :394-421.
#pragma once
#include "common.cuh"

namespace ts {

// Decision for one request given the three cosine terms.  Thread 0 of the block calls it.
// The request's flag, and the caller's copy of it when one was asked for (written by the kernel itself: a copy
// node between the kernels of a captured token would serialise them).
__device__ __forceinline__ void put_flag(const LayerParams& p, int b, int f) {
    p.flags[b] = f;
    if (p.flags_out != nullptr) p.flags_out[b] = f;
}

template <typename T>
__device__ __forceinline__ int decide(const LayerParams& p, int b, int req, float dot, float qq, float cc) {
    int flag = TS_FLAG_RECOMPUTE;
    if (p.query_cache) {
        int* valid = p.valid + (size_t)req * p.n_layers + p.layer;
        bool recompute = true;
        if (*valid) {
            // cos = dot / (sqrt(qq) * sqrt(cc)), every operation rounded to fp32
            float den = __fmul_rn(__fsqrt_rn(qq), __fsqrt_rn(cc));
            float c = (den == 0.f) ? 0.f : __fdiv_rn(dot, den);
            recompute = c < p.theta;                       // strict <, :397-400
        }
        flag = recompute ? TS_FLAG_RECOMPUTE : TS_FLAG_REUSE;
        atomicAdd(p.counters + 2 * (size_t)req, 1ULL);     // retrieval_count, :421
        if (!recompute) atomicAdd(p.counters + 2 * (size_t)req + 1, 1ULL);  // skip_count, :420
        if (recompute) *valid = 1;                         // is_first_query = False, :417
    }
    return flag;
}

struct PrepShared {
    int flag;
    float terms[3];
};

// A group of `nthr` consecutive threads of the CTA (all of them, or some of its warps) that synchronises
// on hardware barrier `bar`; `tid` is the thread's index inside the group.
struct ThreadGroup {
    int tid, nthr, bar;
    __device__ __forceinline__ void sync() const {
        asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(nthr) : "memory");
    }
};
__device__ __forceinline__ ThreadGroup whole_cta() { return ThreadGroup{(int)threadIdx.x, (int)blockDim.x, 0}; }

// All threads of the group call this for request b (uniformly).  kFusedDecide: decide and update the
// cache here; otherwise only publish the cosine terms (they are summed over ranks first).
template <typename T, bool kFusedDecide>
__device__ __forceinline__ void prepare_request(const LayerParams& p, int b, PrepShared& ps, const ThreadGroup& tg) {
    const int tid = tg.tid;
    int& s_flag = ps.flag;
    float* s_terms = ps.terms;

    const int n = p.seq_lens[b];
    const int req = p.req_pool_indices[b];
    const int hd = p.hq * p.d;
    if (n < 1 || n > p.max_ctx || req < 0 || req >= p.max_reqs) {
        if (tid == 0) { set_error(p.err, TS_ERR_BAD_LENGTH, n); put_flag(p, b, TS_FLAG_DENSE); }
        return;
    }

    // 1. append this step's K/V rows to the pools (:849-850)
    if (p.k_new != nullptr) {
        int loc = p.out_cache_loc[b];
        if (loc < 0 || loc >= p.pool_rows) {
            if (tid == 0) { set_error(p.err, TS_ERR_BAD_SLOT, loc); put_flag(p, b, TS_FLAG_DENSE); }
            return;
        }
        const int row_vec = p.hkv * p.d * (int)sizeof(T) / 16;
        const uint4* ks = reinterpret_cast<const uint4*>(p.k_new) + (size_t)b * row_vec;
        const uint4* vs = reinterpret_cast<const uint4*>(p.v_new) + (size_t)b * row_vec;
        uint4* kd = reinterpret_cast<uint4*>(p.k_pool) + (size_t)loc * row_vec;
        uint4* vd = reinterpret_cast<uint4*>(p.v_pool) + (size_t)loc * row_vec;
#pragma unroll 1
        for (int i = tid; i < row_vec; i += tg.nthr) { kd[i] = ks[i]; vd[i] = vs[i]; }
    }

    // 2. clear this request's first-level histogram and candidate counter
#pragma unroll 1
    for (int i = tid; i < kHistBins; i += tg.nthr) p.hist[(size_t)b * kHistBins + i] = 0u;
    if (tid == 0) p.cand_count[b] = 0u;

    // 3. guard (:376-378): short requests attend to everything
    if (p.n_sel >= n) {
        if (tid == 0) put_flag(p, b, TS_FLAG_DENSE);
        return;
    }

    // 4. rotate the scoring query at the fixed position and round to the model dtype (:98-107).
    //    out[i] = x[i]*cos + (-x[i+d/2])*sin ; out[i+d/2] = x[i+d/2]*cos + x[i]*sin, each product and
    //    the sum rounded separately, as eager tensor arithmetic does.
    const T* q = reinterpret_cast<const T*>(p.q) + (size_t)b * hd;
    T* qr = reinterpret_cast<T*>(p.q_rot) + (size_t)b * hd;
    const int half = p.d / 2;
#pragma unroll 1
    for (int e = tid; e < p.hq * half; e += tg.nthr) {
        int h = e / half, i = e % half;
        if (p.q_prerot) {                                  // a prefill chunk's fingerprint: copy
            qr[h * p.d + i] = q[h * p.d + i];
            qr[h * p.d + i + half] = q[h * p.d + i + half];
            continue;
        }
        float x1 = to_f32<T>(q[h * p.d + i]);
        float x2 = to_f32<T>(q[h * p.d + i + half]);
        float2 cs = p.score_cs[i];
        float r1 = __fadd_rn(__fmul_rn(x1, cs.x), __fmul_rn(-x2, cs.y));
        float r2 = __fadd_rn(__fmul_rn(x2, cs.x), __fmul_rn(x1, cs.y));
        qr[h * p.d + i] = from_f32<T>(r1);
        qr[h * p.d + i + half] = from_f32<T>(r2);
    }
    tg.sync();

    // 5. cosine terms against the cached query in a fixed order: lane j sums elements j + 32*i in
    //    ascending i, then an XOR butterfly (16, 8, 4, 2, 1) joins the 32 partial sums.
    const T* fp = reinterpret_cast<const T*>(p.fp_cache) + ((size_t)req * p.n_layers + p.layer) * hd;
    if (p.query_cache) {
        // every thread pulls a line of the two operand rows into L1 first: the one warp that sums them in the fixed
        // order then waits for L1 instead of L2 on each of its batches
        constexpr int kLine = 128 / (int)sizeof(T);
#pragma unroll 1
        for (int e = tid * kLine; e < hd; e += tg.nthr * kLine) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(fp + e));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(qr + e));
        }
    }
    if (p.query_cache && tid < 32) {
        float dot = 0.f, qq = 0.f, cc = 0.f;
        const bool have = p.valid[(size_t)req * p.n_layers + p.layer] != 0;
        if (have) {
            // sixteen elements per lane are requested together (the sums stay in ascending order): this warp is
            // on the critical path of every layer when the cache is on, and one round trip per element would
            // cost it tens of microseconds
            constexpr int kBatch = 16;
#pragma unroll 1
            for (int e0 = tid; e0 < hd; e0 += 32 * kBatch) {
                float a[kBatch], c[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int e = e0 + 32 * u;
                    const bool in = e < hd;
                    a[u] = in ? to_f32<T>(qr[e]) : 0.f;
                    c[u] = in ? to_f32<T>(fp[e]) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    if (e0 + 32 * u < hd) {
                        dot = __fadd_rn(dot, __fmul_rn(a[u], c[u]));
                        qq = __fadd_rn(qq, __fmul_rn(a[u], a[u]));
                        cc = __fadd_rn(cc, __fmul_rn(c[u], c[u]));
                    }
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                dot = __fadd_rn(dot, __shfl_xor_sync(0xffffffffu, dot, o));
                qq = __fadd_rn(qq, __shfl_xor_sync(0xffffffffu, qq, o));
                cc = __fadd_rn(cc, __shfl_xor_sync(0xffffffffu, cc, o));
            }
        }
        if (tid == 0) {
            s_terms[0] = dot; s_terms[1] = qq; s_terms[2] = cc;
            if (!kFusedDecide) {
                p.cos_terms[4 * b + 0] = dot; p.cos_terms[4 * b + 1] = qq;
                p.cos_terms[4 * b + 2] = cc;  p.cos_terms[4 * b + 3] = 0.f;
            }
        }
    }
    if (!kFusedDecide) {
        if (tid == 0) put_flag(p, b, TS_FLAG_RECOMPUTE);   // provisional: decide_kernel overwrites it
        return;
    }
    tg.sync();

    // 6. decision and cache update (:395-421)
    if (tid == 0) {
        int f = decide<T>(p, b, req, s_terms[0], s_terms[1], s_terms[2]);
        put_flag(p, b, f);
        s_flag = f;
    }
    tg.sync();
    if (p.query_cache && s_flag == TS_FLAG_RECOMPUTE) {    // query_fingerprints_cache[layer] = q (:416)
        T* fpw = reinterpret_cast<T*>(p.fp_cache) + ((size_t)req * p.n_layers + p.layer) * hd;
#pragma unroll 1
        for (int e = tid; e < hd; e += tg.nthr) fpw[e] = qr[e];
    }
}

// Tensor-parallel form: the cosine terms were summed over ranks by the caller.
template <typename T>
__device__ __forceinline__ void decide_request(const LayerParams& p, int b, PrepShared& ps) {
    const int tid = threadIdx.x;
    int& s_flag = ps.flag;
    const int n = p.seq_lens[b];
    const int req = p.req_pool_indices[b];
    if (n < 1 || n > p.max_ctx || req < 0 || req >= p.max_reqs) return;
    if (p.n_sel >= n) return;                              // prep already wrote TS_FLAG_DENSE
    const int hd = p.hq * p.d;
    if (tid == 0) {
        int f = decide<T>(p, b, req, p.cos_terms[4 * b], p.cos_terms[4 * b + 1], p.cos_terms[4 * b + 2]);
        put_flag(p, b, f);
        s_flag = f;
    }
    __syncthreads();
    if (p.query_cache && s_flag == TS_FLAG_RECOMPUTE) {
        const T* qr = reinterpret_cast<const T*>(p.q_rot) + (size_t)b * hd;
        T* fpw = reinterpret_cast<T*>(p.fp_cache) + ((size_t)req * p.n_layers + p.layer) * hd;
#pragma unroll 1
        for (int e = tid; e < hd; e += blockDim.x) fpw[e] = qr[e];
    }
}

}  // namespace ts
