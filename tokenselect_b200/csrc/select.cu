// Exact top-k over the vote vector, union with the init and local windows, position -> pool-row map.
//
// Replaces torch.topk + torch.sort (token_retrieval.py:371-372), the "+ n_init" shift (:433), the
// concatenation init || top-k || local (:436-446), the slot gather (:448), the cached-index reuse
// (:419) / cache write (:415) of the selection cache and get_all_tokens (:329-330) for the dense
// fallback.  Output order is ascending logical position, which the attention's positional rotation
// depends on.
//
// Method (one 1024-thread CTA per request): radix select on the raw fp32 bit pattern (votes are
// >= 0, so unsigned order == value order).  Level 1 uses the 2048-bin histogram of bits [30:20]
// built by the vote pass.  One sweep over the votes then sets a bitmap bit for every candidate above
// the threshold bin and collects the candidates inside it; those are resolved by further radix
// levels on (low 20 vote bits, inverted position), which makes every key distinct and breaks exact
// ties in favour of the lowest position.  A popcount scan of the bitmap emits the winners in
// ascending position.
#include "common.cuh"

namespace ts {

constexpr int kSelThreads = 1024;

struct SelectShared {
    Plan plan;
    unsigned hist[kHistBins];
    unsigned warp_sum[32];
    int res_bin;
    unsigned res_above, res_cnt;
    unsigned cand_count;
};

__device__ __forceinline__ unsigned block_inclusive_scan(unsigned v, unsigned* warp_sum) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        unsigned t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned w = warp_sum[lane];
        unsigned winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            unsigned t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        warp_sum[lane] = winc - w;    // exclusive prefix of the warp totals
    }
    __syncthreads();
    unsigned r = inc + warp_sum[warp];
    __syncthreads();
    return r;
}

// Given a 2048-bin histogram in shared memory, find the bin holding the k-th largest key (bins
// counted from the top), the number of keys in higher bins and the bin's own count.
__device__ __forceinline__ void find_threshold(SelectShared& sh, unsigned k) {
    const int tid = threadIdx.x;
    const unsigned a = sh.hist[kHistBins - 1 - 2 * tid];
    const unsigned c = sh.hist[kHistBins - 2 - 2 * tid];
    const unsigned incl = block_inclusive_scan(a + c, sh.warp_sum);
    const unsigned ex = incl - (a + c);
    if (ex < k && k <= ex + a) {
        sh.res_bin = kHistBins - 1 - 2 * tid; sh.res_above = ex; sh.res_cnt = a;
    } else if (ex + a < k && k <= incl) {
        sh.res_bin = kHistBins - 2 - 2 * tid; sh.res_above = ex + a; sh.res_cnt = c;
    }
    __syncthreads();
}

__device__ __forceinline__ unsigned long long cand_key(uint2 c) {
    return ((unsigned long long)(c.y & 0xFFFFFu) << 32) | (unsigned long long)(0xFFFFFFFFu - c.x);
}

__device__ __forceinline__ int checked_slot(const LayerParams& p, const int* row, int pos) {
    int s = __ldg(row + pos);
    if ((unsigned long long)(long long)s >= (unsigned long long)p.pool_rows) {
        set_error(p.err, TS_ERR_BAD_SLOT, s);
        s = 0;
    }
    return s;
}

__global__ void __launch_bounds__(kSelThreads) select_kernel(const LayerParams p) {
    __shared__ SelectShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!build_plan(p, sh.plan)) return;

    const int b = blockIdx.x;
    const int n = sh.plan.n[b];
    const int flag = sh.plan.flag[b];
    const int req = p.req_pool_indices[b];
    if (n < 1 || n > p.max_ctx || req < 0 || req >= p.max_reqs) return;
    const int* row = p.rtt + (long long)req * p.rtt_stride;
    int* out_slots = p.sel_slots + (size_t)b * p.n_sel;
    int* out_pos = p.sel_pos + (size_t)b * p.n_sel;
    const int k = p.top_k;

    if (flag == TS_FLAG_DENSE) {                       // every token, position order (:329-330)
        for (int i = tid; i < n; i += kSelThreads) { out_pos[i] = i; out_slots[i] = checked_slot(p, row, i); }
        if (tid == 0) p.sel_count[b] = n;
        return;
    }

    int* cache_pos = p.pos_cache + ((size_t)req * p.n_layers + p.layer) * k;
    // init and local windows (:438-444)
    for (int i = tid; i < p.n_init; i += kSelThreads) { out_pos[i] = i; out_slots[i] = checked_slot(p, row, i); }
    for (int i = tid; i < p.n_local; i += kSelThreads) {
        int pos = n - p.n_local + i;
        out_pos[p.n_init + k + i] = pos;
        out_slots[p.n_init + k + i] = checked_slot(p, row, pos);
    }
    if (tid == 0) p.sel_count[b] = p.n_sel;

    if (flag == TS_FLAG_REUSE) {                       // cached positions (:419)
        for (int i = tid; i < k; i += kSelThreads) {
            int pos = cache_pos[i];
            out_pos[p.n_init + i] = pos;
            out_slots[p.n_init + i] = checked_slot(p, row, pos);
        }
        return;
    }

    // ---------------- recompute: exact top-k ----------------
    const int nc = sh.plan.nc[b];
    const int ne = pooled_len(nc, p.kernel_size);
    const size_t off = (size_t)sh.plan.off[b];
    const float* votes = p.votes_sel + off;
    unsigned* bitmap = p.bitmap + off / 32;
    uint2* cand = p.cand + off;

    // level 1: threshold bin from the vote pass's histogram
    for (int i = tid; i < kHistBins; i += kSelThreads) sh.hist[i] = __ldcg(p.hist + (size_t)b * kHistBins + i);
    if (tid == 0) sh.cand_count = 0u;
    __syncthreads();
    find_threshold(sh, (unsigned)k);
    const unsigned b1 = (unsigned)sh.res_bin;
    const unsigned k1 = (unsigned)k - sh.res_above;      // still to take from the threshold bin
    const unsigned n_b1 = sh.res_cnt;

    // sweep: bitmap of the sure winners, list of the threshold bin's candidates
    const int chunk = kSelThreads * 4;
    for (int base = 0; base < ne; base += chunk) {
        const int t = base + tid * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < ne) v = __ldcg(reinterpret_cast<const float4*>(votes + t));
        const float vv[4] = {v.x, v.y, v.z, v.w};
        unsigned above = 0u, eq = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (t + j < ne) {
                unsigned bin = (__float_as_uint(vv[j]) >> 20) & (kHistBins - 1);
                above |= (bin > b1 ? 1u : 0u) << j;
                eq |= (bin == b1 ? 1u : 0u) << j;
            }
        }
        unsigned w = above << (4 * (lane & 7));
        w |= __shfl_xor_sync(0xffffffffu, w, 1);
        w |= __shfl_xor_sync(0xffffffffu, w, 2);
        w |= __shfl_xor_sync(0xffffffffu, w, 4);
        if ((lane & 7) == 0 && t < ne) bitmap[t >> 5] = w;
        // unordered append of the threshold bin's candidates (warp-aggregated)
        const unsigned cnt = __popc(eq);
        unsigned inc = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            unsigned x = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += x;
        }
        const unsigned total = __shfl_sync(0xffffffffu, inc, 31);
        unsigned wbase = 0u;
        if (total) {
            if (lane == 31) wbase = atomicAdd(&sh.cand_count, total);
            wbase = __shfl_sync(0xffffffffu, wbase, 31);
            unsigned at = wbase + inc - cnt;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (eq & (1u << j)) cand[at++] = make_uint2((unsigned)(t + j), __float_as_uint(vv[j]));
        }
    }
    __syncthreads();
    const unsigned n_c = sh.cand_count;                 // == n_b1 when the histogram matches the votes
    if (n_c != n_b1 && tid == 0) set_error(p.err, TS_ERR_INTERNAL, (int)n_c);

    // further levels on (low 20 vote bits | inverted index): 10, 10, 11, 11, 10 bits from the top
    unsigned long long prefix = 0ull, mask_above = 0ull;
    unsigned k_rem = k1, active = n_c;
    const int shifts[5] = {42, 32, 21, 10, 0};
    const unsigned widths[5] = {10, 10, 11, 11, 10};
#pragma unroll 1
    for (int lv = 0; lv < 5; ++lv) {
        if (k_rem >= active) break;                     // everything still active is taken
        for (int i = tid; i < kHistBins; i += kSelThreads) sh.hist[i] = 0u;
        __syncthreads();
        const unsigned long long dmask = (1ull << widths[lv]) - 1ull;
        for (unsigned i = tid; i < n_c; i += kSelThreads) {
            unsigned long long key = cand_key(__ldcg(cand + i));
            if ((key & mask_above) == prefix) atomicAdd(&sh.hist[(unsigned)((key >> shifts[lv]) & dmask)], 1u);
        }
        __syncthreads();
        find_threshold(sh, k_rem);
        prefix |= (unsigned long long)(unsigned)sh.res_bin << shifts[lv];
        mask_above |= dmask << shifts[lv];
        k_rem -= sh.res_above;
        active = sh.res_cnt;
        __syncthreads();
    }
    for (unsigned i = tid; i < n_c; i += kSelThreads) {
        uint2 c = __ldcg(cand + i);
        if ((cand_key(c) & mask_above) >= prefix) atomicOr(bitmap + (c.x >> 5), 1u << (c.x & 31));
    }
    __syncthreads();

    // ordered emit: popcount scan over the bitmap words
    const int words = (ne + 31) / 32;
    const int wpt = (words + kSelThreads - 1) / kSelThreads;
    const int w0 = tid * wpt, w1 = min(w0 + wpt, words);
    unsigned mine = 0u;
    for (int w = w0; w < w1; ++w) mine += __popc(__ldcg(bitmap + w));
    const unsigned incl = block_inclusive_scan(mine, sh.warp_sum);
    unsigned rank = incl - mine;
    if (tid == kSelThreads - 1 && incl != (unsigned)k) set_error(p.err, TS_ERR_INTERNAL, (int)incl);
    for (int w = w0; w < w1; ++w) {
        unsigned bits = __ldcg(bitmap + w);
        while (bits) {
            const int bit = __ffs(bits) - 1;
            bits &= bits - 1;
            const int pos = p.n_init + w * 32 + bit;
            if (rank < (unsigned)k) {
                out_pos[p.n_init + rank] = pos;
                out_slots[p.n_init + rank] = checked_slot(p, row, pos);
                if (p.query_cache) cache_pos[rank] = pos;      // topk_indices_cache[layer] = ... (:415)
            }
            ++rank;
        }
    }
}

cudaError_t launch_select(const LayerParams& p, const Launch& l) {
    select_kernel<<<p.batch, kSelThreads, 0, l.stream>>>(p);
    ++*l.launch_count;
    return cudaGetLastError();
}

}  // namespace ts
