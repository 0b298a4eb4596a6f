// Tail of the layer-step kernel: exact top-k from the votes and, where the shape allows, the sparse
// attention itself, inside the persistent selection kernel (included by fused.cu).
//
//   phase 3  classify   every CTA reads the request's vote histogram, finds the bin of the k-th vote and
//                       sorts its own candidates into sure winners (above the bin), members of the bin and
//                       losers; it publishes ONE record per (request, CTA): the number of sure winners and
//                       the bin's members (inline when they are few, in a global list otherwise).  When the
//                       CTA's possible winners are few, their key and value rows are requested now, before
//                       the selection is final, so that they are in shared memory when the ranks are known.
//   phase 4  resolve    after a grid barrier every CTA reads the records of the CTAs that share the request:
//                       the members of the bin are ranked on (low vote bits, inverted index), which settles
//                       the set; the sure-winner counts of the CTAs in front give the list position of the
//                       CTA's first winner.  Positions and pool rows of the winners are written out.
//   phase 5  attend     every CTA attends to ITS OWN winners plus its share of the rows that never depended
//                       on votes (initial and local windows; whole lists of requests that reuse a cached set
//                       or attend to everything): rows of 16 per warp and KV head on mma.sync, the query at
//                       position count-1, the row at its list position.  One partial (max, sum, output) per
//                       (request, CTA).
//   phase 6  merge      after a last grid barrier the partials of a (request, head, quarter of the head
//                       dimension) are merged by one CTA each and the output row is written.
//
// Replaces, from patcher/token_retrieval.py: topk + sort (:371-372), the "+ n_init" shift (:433),
// init || top-k || local (:436-446), the slot gather (:448), the cache write (:415) and the paged decode
// attention call (:815-825, planned at :802-813).
#pragma once

namespace ts {

constexpr int kRecInline = 12;               // members of the threshold bin a record holds itself
constexpr unsigned kRecOverflow = 0x80000000u;
constexpr int kAttnRowsMax = 64;             // rows one attention round stages in shared memory
constexpr int kMaxGrid = 256;
constexpr int kDirectRankMax = 128;          // members ranked by direct comparison up to this many

struct alignas(128) SelRecord {
    unsigned sure;                           // winners above the threshold bin in this CTA's range
    unsigned n_members;                      // members of the bin in the range (| kRecOverflow: in the global list)
    uint2 members[15];                       // (candidate index, vote bits); the first kRecInline are used
};
static_assert(sizeof(SelRecord) == 128, "one record is one 128-byte line");

// Scratch of phases 3-6; overlays FusedShared::idx, which only the scoring phase and the statistics merge use.
struct TailScratch {
    int row_slot[kAttnRowsMax];              // pool row of a staged attention row
    int row_rank[kAttnRowsMax];              // its list position (rotation angle); < 0: not attended
    int row_t[kAttnRowsMax];                 // candidate index of a possible winner staged early
    unsigned row_v[kAttnRowsMax];            // its vote bits
    float inv_freq[64];                      // rotation frequencies of the attention positions
    unsigned rec_sure[kMaxGrid];
    unsigned rec_off[kMaxGrid];
    unsigned long long kv_bar;               // mbarrier of the staged K/V rows
    unsigned long long key_at;               // key of the k1-th member (direct ranking)
    int fast, fast_static, fast_pot, fast_b;
    unsigned n_inl, n_ovf, sure_before, pad;
};
static_assert(sizeof(TailScratch) <= 2 * kIdxBlock * sizeof(int), "tail scratch must fit the index staging area");

__device__ __forceinline__ TailScratch& tail_scratch(FusedShared& sh) { return *reinterpret_cast<TailScratch*>(&sh.idx[0][0]); }

// Rows per attention round and warps that work on them, per KV heads on this rank.
template <int HKV> struct AttnGeom {
    static constexpr int kRows = HKV >= 4 ? 32 : 64;
    static constexpr int kBlocks = kRows / 16;
    static constexpr int kWarpsBusy = kBlocks * HKV;                 // 16, 8, 8, 4
    static constexpr int kRowB = HKV * 256, kRowS = kRowB + 16;      // row bytes in the pool / padded in shared memory
    static constexpr int kKvBytes = 2 * kRows * kRowS;
    static constexpr int kCsOff = (kKvBytes + 127) / 128 * 128;
    static constexpr int kCsBytes = kRows / 8 * 4096;
    static constexpr int kPartOff = kCsOff + kCsBytes;
    static_assert(kWarpsBusy <= kFusedThreads / 32, "more warps than the CTA has");
};
__device__ __forceinline__ int attn_part_bytes(int warps_busy, int group) { return warps_busy * group * (128 + 2) * 4; }

// First and last CTA that own candidates of request b (nc[b] > 0).
__device__ __forceinline__ void owner_range(const LayerParams& p, const FusedShared& sh, int b, int& c0, int& c1) {
    c0 = tile_owner(sh, (unsigned)sh.tile_off[b]);
    c1 = tile_owner(sh, (unsigned)sh.tile_off[b + 1] - 1u);
}

// Rows of request b's list that do not depend on this step's votes, and how many CTAs share them.
//   RECOMPUTE: the initial and local windows, shared by the CTAs that own the request's candidates;
//   REUSE / DENSE: the whole list, shared by `np` CTAs starting at a request-dependent offset.
struct StaticShare {
    int total;       // rows that do not depend on votes
    int np;          // CTAs (= partials) of the request
    int first;       // first CTA of the share (modulo the grid)
    int chunk;       // rows per CTA
};
__device__ __forceinline__ StaticShare static_share(const LayerParams& p, const FusedShared& sh, int b, int rows_per_round) {
    StaticShare s;
    const int n = sh.plan.n[b], flag = sh.plan.flag[b];
    const int req = p.req_pool_indices[b];
    if (n < 1 || n > p.max_ctx || req < 0 || req >= p.max_reqs) { s.total = 0; s.np = 0; s.first = 0; s.chunk = 1; return s; }
    if (flag == TS_FLAG_RECOMPUTE) {
        int c0, c1;
        owner_range(p, sh, b, c0, c1);
        s.total = p.n_init + p.n_local;
        s.np = c1 - c0 + 1;
        s.first = c0;
    } else {
        s.total = flag == TS_FLAG_DENSE ? n : p.n_sel;
        s.np = min(p.grid, (s.total + rows_per_round - 1) / rows_per_round);
        s.first = (int)(((long long)b * 37) % p.grid);
    }
    s.chunk = max(1, (s.total + s.np - 1) / max(s.np, 1));
    return s;
}
// This CTA's place in the share (-1: not part of it).
__device__ __forceinline__ int share_index(const LayerParams& p, const StaticShare& s) {
    if (s.np <= 0) return -1;
    int i = (int)blockIdx.x - s.first;
    if (i < 0) i += p.grid;
    return i < s.np ? i : -1;
}
// List index, logical position of static row `srow` of request b.
__device__ __forceinline__ void static_row(const LayerParams& p, const FusedShared& sh, int b, int srow, int& list_idx, int& pos) {
    const int n = sh.plan.n[b], flag = sh.plan.flag[b];
    if (flag == TS_FLAG_DENSE) { list_idx = srow; pos = srow; return; }
    if (flag == TS_FLAG_RECOMPUTE) list_idx = srow < p.n_init ? srow : srow + p.top_k;
    else list_idx = srow;
    if (list_idx < p.n_init) pos = list_idx;
    else if (list_idx < p.n_init + p.top_k)
        pos = p.pos_cache[((size_t)sh.plan.req[b] * p.n_layers + p.layer) * p.top_k + (list_idx - p.n_init)];
    else pos = n - p.n_local + (list_idx - p.n_init - p.top_k);
}

// Called by all threads before the first use of the tail's scratch.
__device__ __forceinline__ void tail_init(const LayerParams& p, FusedShared& sh) {
    TailScratch& ts = tail_scratch(sh);
    __syncthreads();                                   // the area's previous users are done
    if (threadIdx.x >= 64 && threadIdx.x < 128 && p.attn_inline) ts.inv_freq[threadIdx.x - 64] = p.attn_inv_freq[threadIdx.x - 64];
    if (threadIdx.x == 0) {
        ts.fast = 0; ts.fast_static = 0; ts.fast_pot = 0; ts.fast_b = -1; ts.pad = 0u;
        mbar_init(smem_u32(&ts.kv_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
}

// ------------------------------------------------------------------------------------------
// phase 3
// ------------------------------------------------------------------------------------------
// Vote of own candidate t of segment s: from shared memory when the CTA's votes were kept there.
__device__ __forceinline__ float own_vote(const LayerParams& p, const FusedShared& sh, const float* votes_s, const float* votes_g,
                                          int s, int t) {
    return sh.own_in_smem ? votes_s[sh.seg_off[s] + (t - sh.seg[s].t0)] : __ldcg(votes_g + t);
}

template <int HKV, bool ATTN>
__device__ __forceinline__ void classify_phase(const LayerParams& p, FusedShared& sh, unsigned char* dyn) {
    constexpr bool attn = ATTN;
    using AG = AttnGeom<(HKV > 0 ? HKV : 1)>;
    const int tid = threadIdx.x;
    TailScratch& ts = tail_scratch(sh);
    const float* votes_s = own_votes(dyn);
    const int* slot_s = own_slots(dyn);
    fstamp(p, 4);
    // The first segment's request: this CTA's share of its window rows can be staged together with the
    // possible winners.  Their pool rows are looked up now (the loads travel with the histogram's).
    int st_cnt = 0, st_slot = 0, st_list = -1;
    if (attn && sh.nseg > 0) {
        const int b = sh.seg[0].b;
        const StaticShare ss = static_share(p, sh, b, AG::kRows);
        const int me = share_index(p, ss);
        if (me >= 0) {
            const int s0 = me * ss.chunk, s1 = min(ss.total, s0 + ss.chunk);
            st_cnt = max(0, s1 - s0);
            if (tid < st_cnt && st_cnt <= AG::kRows) {
                int pos;
                static_row(p, sh, b, s0 + tid, st_list, pos);
                st_slot = checked_slot(p, p.rtt + (long long)sh.plan.req[b] * p.rtt_stride, pos);
            }
        }
    }
#pragma unroll 1
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const float* votes_g = p.votes_final + sh.plan.off[sg.b];
        int own0, own1, per;
        own_range(sg.t0, sg.t1, own0, own1, per);
        // the bin of the k-th vote, from the request's histogram
        fstamp(p, 5);
        find_threshold_global(sh, p.hist + (size_t)sg.b * kHistBins, (unsigned)p.top_k);
        fstamp(p, 6);
        const unsigned b1 = (unsigned)sh.res_bin;
        if (tid == 0) { sh.seg_b1[s] = sh.res_bin; sh.seg_above[s] = sh.res_above; sh.seg_cnt[s] = sh.res_cnt; }
        // pass 1: sure winners and members of the bin among the own candidates
        unsigned sure = 0, eq = 0;
#pragma unroll 1
        for (int t = own0; t < own1; ++t) {
            const unsigned bin = vote_bin(own_vote(p, sh, votes_s, votes_g, s, t));
            sure += bin > b1;
            eq += bin == b1;
        }
        const unsigned long long packed = block_inclusive_scan(((unsigned long long)sure << 32) | eq, sh.warp_sum64);
        if (tid == kFusedThreads - 1) { sh.tmp_u[0] = (unsigned)(packed >> 32); sh.tmp_u[1] = (unsigned)packed; }
        __syncthreads();
        fstamp(p, 7);
        const unsigned sure_tot = sh.tmp_u[0], eq_tot = sh.tmp_u[1];
        const bool overflow = eq_tot > (unsigned)kRecInline;
        SelRecord* rec = p.records + (size_t)sg.b * p.grid + blockIdx.x;
        if (tid == 0) {
            rec->sure = sure_tot;
            rec->n_members = overflow ? (kRecOverflow | eq_tot) : eq_tot;
            sh.tmp_u[2] = overflow ? atomicAdd(p.cand_count + sg.b, eq_tot) : 0u;
        }
        const bool fast = attn && s == 0 && sh.own_in_smem && st_cnt <= AG::kRows &&
                          (unsigned)st_cnt + sure_tot + eq_tot <= (unsigned)AG::kRows;
        __syncthreads();
        // pass 2: the members go into the record (or the list); possible winners are staged
        unsigned m_at = (unsigned)packed - eq;                                   // members in front of this thread's
        unsigned p_at = (unsigned)(packed >> 32) - sure + m_at;                  // possible winners in front of it
        uint2* list = p.cand + sh.plan.off[sg.b] + sh.tmp_u[2];
#pragma unroll 1
        for (int t = own0; t < own1; ++t) {
            const float v = own_vote(p, sh, votes_s, votes_g, s, t);
            const unsigned bin = vote_bin(v);
            if (bin == b1) {
                const uint2 m = make_uint2((unsigned)t, __float_as_uint(v));
                if (overflow) list[m_at] = m; else rec->members[m_at] = m;
                ++m_at;
            }
            if (fast && bin >= b1) {
                const int r = st_cnt + (int)p_at++;
                ts.row_t[r] = t;
                ts.row_v[r] = __float_as_uint(v);
                ts.row_slot[r] = slot_s[sh.seg_off[s] + (t - sg.t0)];
                ts.row_rank[r] = -2;
            }
        }
        if (fast) {
            if (tid < st_cnt) { ts.row_slot[tid] = st_slot; ts.row_rank[tid] = st_list; }
            if (tid == 0) { ts.fast = 1; ts.fast_static = st_cnt; ts.fast_pot = (int)(sure_tot + eq_tot); ts.fast_b = sg.b; }
        }
        __syncthreads();
        fstamp(p, 8);
    }
    fstamp(p, 9);
}

// Requests the rows classify_phase staged.  Called after the CTA has ARRIVED at the grid barrier that follows
// the classification (the copy engine takes ~35 ns per row copy to issue; the other CTAs need not wait for that)
// and before it waits there: the rows land during the wait.
template <int HKV>
__device__ __forceinline__ void issue_staged_rows(const LayerParams& p, FusedShared& sh, unsigned char* dyn) {
    using AG = AttnGeom<HKV>;
    const int tid = threadIdx.x;
    TailScratch& ts = tail_scratch(sh);
    if (ts.fast) {
        const int rows = ts.fast_static + ts.fast_pot;
        const uint32_t kbase = smem_u32(dyn), vbase = kbase + AG::kRows * AG::kRowS;
        const uint32_t bar = smem_u32(&ts.kv_bar);
        asm volatile("fence.proxy.async;" ::: "memory");
        if (tid == 0) mbar_expect_tx(bar, (uint32_t)rows * 2u * AG::kRowB);
        if (tid < rows) {
            const int slot = ts.row_slot[tid];
            bulk_g2s(kbase + tid * AG::kRowS, reinterpret_cast<const unsigned char*>(p.k_pool) + (size_t)slot * AG::kRowB, AG::kRowB, bar);
            bulk_g2s(vbase + tid * AG::kRowS, reinterpret_cast<const unsigned char*>(p.v_pool) + (size_t)slot * AG::kRowB, AG::kRowB, bar);
        }
    }
}

// Where the threshold bin's members are staged when the attention's inputs are prepared early: behind the
// partial outputs, running into the shared-memory copies of the CTA's own votes and pool rows (no longer
// needed once the possible winners are staged).
template <int HKV>
__device__ __forceinline__ int early_cand_offset(const LayerParams& p) {
    using AG = AttnGeom<HKV>;
    return (AG::kPartOff + attn_part_bytes(AG::kWarpsBusy, p.group) + 15) & ~15;
}

template <int HKV> __device__ __forceinline__ void attend_prepare(const LayerParams& p, FusedShared& sh, unsigned char* dyn, int b,
                                                                  int rows, int cs_rows, int tid0, int nthr);

// While the CTA waits at the grid barrier after the classification: everything the attention over the staged
// rows needs except the winners' final list positions (rotated query, zeros in unused rows, rotation rows of the
// window rows).  Only when the members of all records are sure to fit their alternative staging place.
template <int HKV>
__device__ __forceinline__ void early_prepare(const LayerParams& p, FusedShared& sh, unsigned char* dyn) {
    TailScratch& ts = tail_scratch(sh);
    if (ts.fast == 0 || sh.nseg != 1) return;     // (a second segment would still read the own-vote copies)
    int c0, c1;
    owner_range(p, sh, ts.fast_b, c0, c1);
    const int room = (kFusedDynSmem - early_cand_offset<HKV>(p)) / 8;
    if ((c1 - c0 + 1) * kRecInline > room) return;
    attend_prepare<HKV>(p, sh, dyn, ts.fast_b, ts.fast_static + ts.fast_pot, ts.fast_static, 0, kFusedThreads);
    if (threadIdx.x == 0) ts.pad = 1u;
}

// ------------------------------------------------------------------------------------------
// phase 4
// ------------------------------------------------------------------------------------------
struct Resolved {
    unsigned long long prefix, mask;     // a member is selected iff (key & mask) >= prefix
    unsigned before;                     // winners of the request in front of this CTA's range
    unsigned b1;
};

// Gathers the records of the CTAs that share request sg.b, settles which members of the threshold bin are
// selected and counts the winners in front of this CTA's candidates.  cand_s: staging for the members.
__device__ __forceinline__ Resolved resolve_segment(const LayerParams& p, FusedShared& sh, int s, uint2* cand_s, unsigned cand_cap) {
    const int tid = threadIdx.x;
    TailScratch& ts = tail_scratch(sh);
    const Seg sg = sh.seg[s];
    int c0, c1;
    owner_range(p, sh, sg.b, c0, c1);
    const int nown = c1 - c0 + 1;
    const SelRecord* recs = p.records + (size_t)sg.b * p.grid + c0;
    fstamp(p, 10);
    // headers, and the overflow list's length
    unsigned ovf = 0;
    if (tid < nown) {
        // a CTA inside the range may own no tile at all (fewer tiles than CTAs): it wrote no record
        const unsigned c = (unsigned)(c0 + tid);
        const int lo = max((int)tile_lo(sh, c), sh.tile_off[sg.b]);
        const int hi = min((int)tile_lo(sh, c + 1u), sh.tile_off[sg.b + 1]);
        uint2 h = make_uint2(0u, 0u);
        if (lo < hi) h = __ldcg(reinterpret_cast<const uint2*>(recs + tid));
        ts.rec_sure[tid] = h.x;
        ts.rec_off[tid] = h.y;
    }
    if (tid == kFusedThreads - 1) ovf = __ldcg(p.cand_count + sg.b);
    __syncthreads();
    fstamp(p, 11);
    if (tid < 32) {
        // exclusive prefix of the inline member counts; sure winners of the CTAs in front
        unsigned carry = 0, sb = 0;
#pragma unroll 1
        for (int base = 0; base < nown; base += 32) {
            const int i = base + tid;
            const unsigned nm = i < nown ? ts.rec_off[i] : 0u;
            const unsigned inl = (nm & kRecOverflow) ? 0u : nm;
            unsigned inc = inl;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned t = __shfl_up_sync(0xffffffffu, inc, o);
                if (tid >= o) inc += t;
            }
            if (i < nown) {
                ts.rec_off[i] = carry + inc - inl;
                if (c0 + i < (int)blockIdx.x) sb += ts.rec_sure[i];
                ts.rec_sure[i] = inl;                    // from here on: the record's inline member count
            }
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) sb += __shfl_xor_sync(0xffffffffu, sb, o);
        if (tid == 0) { ts.n_inl = carry; ts.sure_before = sb; }
    }
    if (tid == kFusedThreads - 1) ts.n_ovf = ovf;
    __syncthreads();
    fstamp(p, 12);
    const unsigned n_inl = ts.n_inl, n_ovf = ts.n_ovf, n_c = n_inl + n_ovf;
    // members: the inline ones always fit the staging area; the list's part when there is room
#pragma unroll 1
    for (int i = tid; i < nown * kRecInline; i += kFusedThreads) {
        const int r = i / kRecInline, m = i - r * kRecInline;
        if ((unsigned)m < ts.rec_sure[r]) cand_s[ts.rec_off[r] + m] = __ldcg(&recs[r].members[m]);
    }
    const uint2* cand_g = p.cand + sh.plan.off[sg.b];
    const bool staged = n_c <= cand_cap;
    if (staged)
#pragma unroll 1
        for (unsigned i = tid; i < n_ovf; i += kFusedThreads) cand_s[n_inl + i] = __ldcg(cand_g + i);
    __syncthreads();
    auto get_cand = [&](unsigned i) -> uint2 { return (i < n_inl || staged) ? cand_s[i] : __ldcg(cand_g + (i - n_inl)); };
    fstamp(p, 13);

    Resolved r;
    r.b1 = (unsigned)sh.seg_b1[s];
    const unsigned k1 = (unsigned)p.top_k - sh.seg_above[s];     // 1 <= k1 <= n_c members still to take
    unsigned long long prefix = 0ull, mask_above = 0ull;
    if (k1 >= n_c) {
        // every member is taken
    } else if (n_c <= (unsigned)kDirectRankMax) {
        // few members: the one with exactly k1-1 larger keys is the last one taken
        if (tid < (int)n_c) {
            const unsigned long long key = cand_key(cand_s[tid]);
            unsigned larger = 0;
#pragma unroll 1
            for (unsigned j = 0; j < n_c; ++j) larger += cand_key(cand_s[j]) > key;
            if (larger == k1 - 1) ts.key_at = key;
        }
        __syncthreads();
        prefix = ts.key_at;
        mask_above = ~0ull;
    } else {
        // radix levels on (low 20 vote bits | inverted index): 10, 10, 11, 11, 10 bits from the top
        unsigned k_rem = k1, active = n_c;
        const int shifts[5] = {42, 32, 21, 10, 0};
        const unsigned widths[5] = {10, 10, 11, 11, 10};
#pragma unroll 1
        for (int lv = 0; lv < 5; ++lv) {
            if (k_rem >= active) break;                    // everything still active is taken
            __syncthreads();
#pragma unroll 1
            for (int i = tid; i < kHistBins; i += kFusedThreads) sh.hist[i] = 0u;
            __syncthreads();
            const unsigned long long dmask = (1ull << widths[lv]) - 1ull;
#pragma unroll 1
            for (unsigned i = tid; i < n_c; i += kFusedThreads) {
                const unsigned long long key = cand_key(get_cand(i));
                if ((key & mask_above) == prefix) atomicAdd(&sh.hist[(unsigned)((key >> shifts[lv]) & dmask)], 1u);
            }
            __syncthreads();
            find_threshold(sh, k_rem);
            prefix |= (unsigned long long)(unsigned)sh.res_bin << shifts[lv];
            mask_above |= dmask << shifts[lv];
            k_rem -= sh.res_above;
            active = sh.res_cnt;
        }
    }
    fstamp(p, 14);
    // selected members in front of this CTA's range
    unsigned before = 0;
#pragma unroll 1
    for (unsigned i = tid; i < n_c; i += kFusedThreads) {
        const uint2 c = get_cand(i);
        if ((int)c.x < sg.t0 && (cand_key(c) & mask_above) >= prefix) ++before;
    }
    __syncthreads();                                       // cand_s may be reused by the caller after this
    const unsigned long long tot = block_inclusive_scan((unsigned long long)before, sh.warp_sum64);
    if (tid == kFusedThreads - 1) sh.tmp_u[3] = (unsigned)tot;
    __syncthreads();
    r.prefix = prefix;
    r.mask = mask_above;
    r.before = ts.sure_before + sh.tmp_u[3];
    fstamp(p, 15);
    return r;
}

__device__ __forceinline__ bool vote_selected(const Resolved& r, int t, unsigned vbits) {
    const unsigned bin = (vbits >> 20) & (kHistBins - 1);
    if (bin > r.b1) return true;
    if (bin < r.b1) return false;
    return (cand_key(make_uint2((unsigned)t, vbits)) & r.mask) >= r.prefix;
}

// Writes the winners of segment s in position order (list index n_init + rank) and leaves, in
// seg_above[s] / seg_cnt[s], the list index of the CTA's first winner and their number.
__device__ __forceinline__ void emit_segment(const LayerParams& p, FusedShared& sh, unsigned char* dyn, int s, const Resolved& r,
                                             bool fast) {
    const int tid = threadIdx.x;
    TailScratch& ts = tail_scratch(sh);
    const Seg sg = sh.seg[s];
    const int k = p.top_k;
    const int req = sh.plan.req[sg.b];
    const int* row = p.rtt + (long long)req * p.rtt_stride;
    int* out_slots = p.sel_slots + (size_t)sg.b * p.n_sel;
    int* out_pos = p.sel_pos + (size_t)sg.b * p.n_sel;
    int* cache_pos = p.pos_cache + ((size_t)req * p.n_layers + p.layer) * k;
    unsigned total_here;
    if (fast) {
        // the possible winners sit in the staged rows, in position order: rank them with one warp
        const int st = ts.fast_static, np = ts.fast_pot;
        if (tid < 32) {
            unsigned carry = 0;
#pragma unroll 1
            for (int base = 0; base < np; base += 32) {
                const int i = base + tid;
                const bool sel = i < np && vote_selected(r, ts.row_t[st + i], ts.row_v[st + i]);
                const unsigned bal = __ballot_sync(0xffffffffu, sel);
                if (i < np) {
                    const unsigned rank = r.before + carry + __popc(bal & ((1u << tid) - 1u));
                    ts.row_rank[st + i] = sel ? (int)(p.n_init + rank) : -1;
                    if (sel) {
                        if (rank < (unsigned)k) {
                            const int pos = p.n_init + ts.row_t[st + i];
                            out_pos[p.n_init + rank] = pos;
                            out_slots[p.n_init + rank] = ts.row_slot[st + i];
                            if (p.query_cache) cache_pos[rank] = pos;          // topk_indices_cache[layer] = ... (:415)
                        } else {
                            set_error(p.err, TS_ERR_INTERNAL, (int)rank);
                        }
                    }
                }
                carry += __popc(bal);
            }
            if (tid == 0) { sh.tmp_u[0] = r.before; sh.tmp_u[1] = carry; }
        }
        __syncthreads();
        total_here = sh.tmp_u[0] + sh.tmp_u[1];
    } else {
        const float* votes_s = own_votes(dyn);
        const float* votes_g = p.votes_final + sh.plan.off[sg.b];
        int own0, own1, per;
        own_range(sg.t0, sg.t1, own0, own1, per);
        unsigned mine = 0;
#pragma unroll 1
        for (int t = own0; t < own1; ++t)
            mine += vote_selected(r, t, __float_as_uint(own_vote(p, sh, votes_s, votes_g, s, t)));
        const unsigned long long packed = block_inclusive_scan((unsigned long long)mine, sh.warp_sum64);
        if (tid == kFusedThreads - 1) { sh.tmp_u[0] = r.before; sh.tmp_u[1] = (unsigned)packed; }
        __syncthreads();
        unsigned rank = r.before + (unsigned)packed - mine;
#pragma unroll 1
        for (int t = own0; t < own1; ++t) {
            if (!vote_selected(r, t, __float_as_uint(own_vote(p, sh, votes_s, votes_g, s, t)))) continue;
            if (rank < (unsigned)k) {
                const int pos = p.n_init + t;
                out_pos[p.n_init + rank] = pos;
                out_slots[p.n_init + rank] = sh.own_in_smem ? own_slots(dyn)[sh.seg_off[s] + (t - sg.t0)] : checked_slot(p, row, pos);
                if (p.query_cache) cache_pos[rank] = pos;
            } else {
                set_error(p.err, TS_ERR_INTERNAL, (int)rank);
            }
            ++rank;
        }
        total_here = sh.tmp_u[0] + sh.tmp_u[1];
    }
    // the CTA owning the request's last candidates checks the total
    if (sg.t1 >= sh.plan.nc[sg.b] && tid == 0 && total_here != (unsigned)k) set_error(p.err, TS_ERR_INTERNAL, (int)total_here);
    __syncthreads();
    if (tid == 0) { sh.seg_above[s] = (unsigned)p.n_init + sh.tmp_u[0]; sh.seg_cnt[s] = sh.tmp_u[1]; }
    __syncthreads();
}

// ------------------------------------------------------------------------------------------
// phase 5: attention over staged rows
// ------------------------------------------------------------------------------------------
// sin and cos of a non-negative angle of up to a few thousand radians: two-constant reduction to [-pi, pi]
// (2*pi = 6.2831854820251465 - 1.7484555e-7 in fp32 pieces), then the special-function unit (absolute error
// below 1e-6, far inside the attention tolerance; the library's sincosf would cost hundreds of instruction
// bytes at each place it is used).
__device__ __forceinline__ void sincos_reduced(float a, float& sn, float& cn) {
    const float n = rintf(a * 0.15915494309189535f);
    float r = fmaf(n, -6.2831854820251465f, a);
    r = fmaf(n, 1.7484555e-7f, r);
    sn = __sinf(r);
    cn = __cosf(r);
}

constexpr int kQStride = 136;            // floats per head of the staged rotated query (8 floats of padding: bank spread)

// Rotation rows of the staged rows' list positions, in the order the lanes of the multiplying warps read them:
// positions in tiles of eight; inside a tile the (cos, sin) of frequency i = 16s + 8u + 2t + w of position g
// sits in float2 (((s*2+u)*8 + g)*4 + t)*2 + w.
__device__ __forceinline__ void fill_rotation_rows(const LayerParams& p, const TailScratch& ts, float2* cs, int row0, int row1,
                                                   int tid0 = 0, int nthr = kFusedThreads) {
#pragma unroll 1
    for (int idx = row0 * 64 + (int)threadIdx.x - tid0; idx < row1 * 64; idx += nthr) {
        const int r = idx >> 6, i = idx & 63;
        const int rank = max(ts.row_rank[r], 0);
        float sn, cn;
        sincos_reduced(__fmul_rn((float)rank, ts.inv_freq[i]), sn, cn);
        const int tile = r >> 3, g = r & 7;
        const int s = i >> 4, u = (i >> 3) & 1, t = (i >> 1) & 3, w = i & 1;
        cs[(tile * 256 + ((s * 2 + u) * 8 + g) * 4 + t) * 2 + w] = make_float2(cn, sn);
    }
}

// The request's query rotated at position count-1, fp32, [hq][kQStride] in shared memory.
__device__ __forceinline__ void fill_rotated_query(const LayerParams& p, const TailScratch& ts, const __nv_bfloat16* q_b, int count,
                                                   float* q_s, int tid0 = 0, int nthr = kFusedThreads) {
#pragma unroll 1
    for (int idx = (int)threadIdx.x - tid0; idx < p.hq * 64; idx += nthr) {
        const int h = idx >> 6, i = idx & 63;
        float sn, cn;
        sincos_reduced(__fmul_rn((float)(count - 1), ts.inv_freq[i]), sn, cn);
        const float x1 = __bfloat162float(q_b[h * 128 + i]), x2 = __bfloat162float(q_b[h * 128 + i + 64]);
        q_s[h * kQStride + i] = x1 * cn - x2 * sn;
        q_s[h * kQStride + i + 64] = x2 * cn + x1 * sn;
    }
}

// What the attention over a round's staged rows needs besides the rows' final list positions: zeros in the
// unused rows of the last, partly filled block (0-weight products must stay finite), "not attended" marks for
// them, the rotated query, and (from row `cs_rows` down) the rotation rows of positions already known.  Run
// by the threads tid0 .. tid0 + nthr - 1.
template <int HKV>
__device__ __forceinline__ void attend_prepare(const LayerParams& p, FusedShared& sh, unsigned char* dyn, int b, int rows,
                                               int cs_rows, int tid0, int nthr) {
    using AG = AttnGeom<HKV>;
    const int t = (int)threadIdx.x - tid0;
    TailScratch& ts = tail_scratch(sh);
    unsigned char* sm_k = dyn;
    unsigned char* sm_v = dyn + AG::kRows * AG::kRowS;
    const int rows16 = (rows + 15) / 16 * 16;
#pragma unroll 1
    for (int i = rows * (AG::kRowB / 16) + t; i < rows16 * (AG::kRowB / 16); i += nthr) {
        const int r = i / (AG::kRowB / 16), c = i - r * (AG::kRowB / 16);
        *reinterpret_cast<uint4*>(sm_k + r * AG::kRowS + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(sm_v + r * AG::kRowS + c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (t >= rows && t < rows16) ts.row_rank[t] = -1;
    const int count = min(sh.plan.n[b], p.n_sel);
    fill_rotated_query(p, ts, reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)b * p.hq * 128, count,
                       reinterpret_cast<float*>(dyn + AG::kPartOff), tid0, nthr);
    if (cs_rows > 0) fill_rotation_rows(p, ts, reinterpret_cast<float2*>(dyn + AG::kCsOff), 0, cs_rows, tid0, nthr);
}

// One warp: S^T of 16 staged rows x one KV head's query heads on mma.sync, rows in groups of eight (the N of
// the instruction); a group without rows is skipped.  The rotated query and keys (fp32) go into the tensor
// cores as fp16: 11 significant bits, i.e. a logit error of a few 1e-4 at these shapes -- an order of magnitude
// inside what the bf16 output rounding already costs -- for ONE instruction per k-step (the bf16 high/low
// split of attend.cu needs three; this path is bound by the tensor pipe's rate for mma.sync).  Values beyond
// the fp16 range saturate.  The loops are kept rolled: this code runs once per launch.
template <int HKV>
__device__ __forceinline__ void attend_scores(const LayerParams& p, const unsigned char* sm_k, const float4* sm_cs,
                                              const float* q_s, int wb, int kv, int rows, float (&sc)[2][4]) {
    using AG = AttnGeom<HKV>;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = p.group;
    const bool on = g < G;
    const float* qh = q_s + (size_t)(kv * G + min(g, G - 1)) * kQStride;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[j][i] = 0.f;
    const int lrow = lane & 7, lsel = lane >> 3;
    const int ngroups = min(2, (rows - wb * 16 + 7) >> 3);        // groups of eight rows this block really has
#pragma unroll 1
    for (int s = 0; s < 4; ++s) {
        // A fragments of k-steps s and s+4 (rows 8..15 of A are unused: zero)
        uint32_t af[2][2];
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const float2 x = *reinterpret_cast<const float2*>(qh + 16 * (s + 4 * k2) + 8 * u + 2 * t);
                af[k2][u] = pack_f16x2_sat(on ? x.x : 0.f, on ? x.y : 0.f);
            }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (j < ngroups) {
                const float4* cst = sm_cs + (size_t)(wb * 2 + j) * 256;
                uint32_t r[4];
                const int doff = 16 * s + (lsel & 1) * 8 + (lsel >> 1) * 64;
                ldmatrix_x4(r, smem_u32(sm_k) + (wb * 16 + 8 * j + lrow) * AG::kRowS + kv * 256 + doff * 2);
                uint32_t bf[2][2];                         // [k-step s | s+4][b0 | b1]
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float4 cs = cst[((s * 2 + u) * 8 + g) * 4 + t];
                    const float x1a = __uint_as_float(r[u] << 16), x1b = __uint_as_float(r[u] & 0xFFFF0000u);
                    const float x2a = __uint_as_float(r[2 + u] << 16), x2b = __uint_as_float(r[2 + u] & 0xFFFF0000u);
                    bf[0][u] = pack_f16x2_sat(x1a * cs.x - x2a * cs.y, x1b * cs.z - x2b * cs.w);
                    bf[1][u] = pack_f16x2_sat(x2a * cs.x + x1a * cs.y, x2b * cs.z + x1b * cs.w);
                }
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {
                    const uint32_t a4[4] = {af[k2][0], 0u, af[k2][1], 0u};
                    mma_f16_16816(sc[j], a4, bf[k2][0], bf[k2][1]);
                }
            }
        }
    }
}

// Softmax numerators of the block (base 2) and O^T = V^T . P^T into part_o [G][128], (max, sum) into part_ml [G].
template <int HKV>
__device__ __forceinline__ void attend_values(const LayerParams& p, const TailScratch& ts, const unsigned char* sm_v, int wb,
                                              int kv, int rows, const float (&sc)[2][4], float* part_o, float2* part_ml) {
    using AG = AttnGeom<HKV>;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = p.group;
    const int lrow = lane & 7;
    float x[2][2], mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            float v = sc[j][u] * p.sm_scale;
            if (p.logit_cap > 0.f) v = p.logit_cap * tanhf(v / p.logit_cap);
            const int rr = wb * 16 + 8 * j + 2 * t + u;
            v = (rr < rows && ts.row_rank[rr] >= 0) ? v * kLog2e : -INFINITY;
            x[j][u] = v;
            mx = fmaxf(mx, v);
        }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    float pe[2][2], lsum = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            pe[j][u] = (x[j][u] == -INFINITY) ? 0.f : ex2_ftz(fmaxf(x[j][u] - mx, -126.f));
            lsum += pe[j][u];
        }
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
    uint32_t ph[2], pl[2];
    split_bf16x2(pe[0][0], pe[0][1], ph[0], pl[0]);
    split_bf16x2(pe[1][0], pe[1][1], ph[1], pl[1]);
#pragma unroll 1
    for (int db = 0; db < 8; ++db) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, smem_u32(sm_v) + (wb * 16 + ((lane >> 4) & 1) * 8 + lrow) * AG::kRowS + kv * 256 +
                                 (16 * db + ((lane >> 3) & 1) * 8) * 2);
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        mma_bf16_16816(o, a, ph[0], ph[1]);
        mma_bf16_16816(o, a, pl[0], pl[1]);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int hh = 2 * t + u;
            if (hh < G) {
                part_o[hh * 128 + 16 * db + g] = o[u];
                part_o[hh * 128 + 16 * db + g + 8] = o[2 + u];
            }
        }
    }
    if (t == 0 && g < G) part_ml[g] = make_float2(mx, lsum);
}

// The rows of one (request, CTA): `st_cnt` rows that never depended on votes starting at static row st0,
// then `own_cnt` winners of this CTA starting at list index own0.  `staged`: all rows are already on their
// way (requested by classify_phase) and listed in the scratch.  Writes partial `pslot` of the request.
template <int HKV>
__device__ __forceinline__ void attend_rowset(const LayerParams& p, FusedShared& sh, unsigned char* dyn, int b, int pslot,
                                              int st0, int st_cnt, int own0, int own_cnt, bool staged, bool prepared,
                                              uint32_t& kv_parity, bool& dead) {
    using AG = AttnGeom<HKV>;
    const int tid = threadIdx.x, warp = tid >> 5;
    TailScratch& ts = tail_scratch(sh);
    const int G = p.group, hq = p.hq;
    unsigned char* sm_k = dyn;
    unsigned char* sm_v = dyn + AG::kRows * AG::kRowS;
    float2* cs = reinterpret_cast<float2*>(dyn + AG::kCsOff);
    float* part = reinterpret_cast<float*>(dyn + AG::kPartOff);       // [warps busy][G][130]; first the rotated query
    const uint32_t bar = smem_u32(&ts.kv_bar);
    const int count = min(sh.plan.n[b], p.n_sel);
    const __nv_bfloat16* q_b = reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)b * hq * 128;
    float* g_o = p.part_o + (size_t)pslot * hq * 128;
    float2* g_ml = p.part_ml + (size_t)pslot * hq;
    const int total = st_cnt + own_cnt;
    if (total == 0) {
#pragma unroll 1
        for (int h = tid; h < hq; h += kFusedThreads) g_ml[h] = make_float2(-INFINITY, 0.f);
        return;
    }
    const int* rtt_row = p.rtt + (long long)sh.plan.req[b] * p.rtt_stride;
#pragma unroll 1
    for (int r0 = 0; r0 < total; r0 += AG::kRows) {
        const int rows = min(AG::kRows, total - r0);
        const int rows16 = (rows + 15) / 16 * 16;
        if (!staged) {
            // look the round's rows up and request them
            __syncthreads();                               // the previous round's readers are done
            if (tid < rows) {
                const int i = r0 + tid;
                int slot, rank;
                if (i < st_cnt) {
                    int pos;
                    static_row(p, sh, b, st0 + i, rank, pos);
                    slot = checked_slot(p, rtt_row, pos);
                } else {
                    rank = own0 + (i - st_cnt);
                    slot = __ldcg(p.sel_slots + (size_t)b * p.n_sel + rank);
                    if ((unsigned long long)(long long)slot >= (unsigned long long)p.pool_rows) {
                        set_error(p.err, TS_ERR_BAD_SLOT, slot);
                        slot = 0;
                    }
                }
                ts.row_slot[tid] = slot;
                ts.row_rank[tid] = rank;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            __syncthreads();
            if (tid == 0) mbar_expect_tx(bar, (uint32_t)rows * 2u * AG::kRowB);
            if (tid < rows) {
                const int slot = ts.row_slot[tid];
                bulk_g2s(smem_u32(sm_k) + tid * AG::kRowS, reinterpret_cast<const unsigned char*>(p.k_pool) + (size_t)slot * AG::kRowB,
                         AG::kRowB, bar);
                bulk_g2s(smem_u32(sm_v) + tid * AG::kRowS, reinterpret_cast<const unsigned char*>(p.v_pool) + (size_t)slot * AG::kRowB,
                         AG::kRowB, bar);
            }
        }
        if (prepared && r0 == 0) {
            // the caller zeroed the unused rows, rotated the query and filled the static rows' rotation rows
            // while the final set was being settled; only the winners' rotation rows are left
            fill_rotation_rows(p, ts, cs, ts.fast_static, rows16);
        } else {
            attend_prepare<HKV>(p, sh, dyn, b, rows, 0, 0, kFusedThreads);
            __syncthreads();
            fill_rotation_rows(p, ts, cs, 0, rows16);
        }
        __syncthreads();
        fstamp(p, 18);
        mbar_wait(bar, kv_parity, p.err, dead, 5, p.wait_cycles);
        kv_parity ^= 1u;
        fstamp(p, 19);
        const int nblk = rows16 / 16;
        const int wb = warp / HKV, kv = warp % HKV;
        float sc[2][4];
        if (wb < nblk) attend_scores<HKV>(p, sm_k, reinterpret_cast<const float4*>(cs), part, wb, kv, rows, sc);
        __syncthreads();                                   // the rotated query has been read: its place takes the partials
        float* my_o = part + (size_t)warp * G * 130;
        if (wb < nblk) attend_values<HKV>(p, ts, sm_v, wb, kv, rows, sc, my_o, reinterpret_cast<float2*>(my_o + G * 128));
        fstamp(p, 20);
        __syncthreads();
        // merge the blocks of the round (and, from the second round on, the partial written so far):
        // per head the new (max, sum) and the weights of the pieces, then the weighted outputs
        float* s_w = reinterpret_cast<float*>(sh.hist);               // [hq][kBlocks + 1] weights, then [hq][2] (max, sum)
        constexpr int kW = AG::kBlocks + 1;
        const bool more = r0 > 0;
        if (tid < hq) {
            const int h = tid, kvh = h / G, gg = h - kvh * G;
            const float2 prev = more ? g_ml[h] : make_float2(-INFINITY, 0.f);
            float mm = prev.x;
#pragma unroll 1
            for (int w = 0; w < nblk; ++w)
                mm = fmaxf(mm, reinterpret_cast<const float2*>(part + (size_t)(w * HKV + kvh) * G * 130 + G * 128)[gg].x);
            const float wp = (prev.x == -INFINITY) ? 0.f : ex2_ftz(fmaxf(prev.x - mm, -126.f));
            float ll = prev.y * wp;
            s_w[h * kW + AG::kBlocks] = wp;
#pragma unroll 1
            for (int w = 0; w < AG::kBlocks; ++w) {
                float wgt = 0.f;
                if (w < nblk) {
                    const float2 ml = reinterpret_cast<const float2*>(part + (size_t)(w * HKV + kvh) * G * 130 + G * 128)[gg];
                    wgt = (ml.x == -INFINITY) ? 0.f : ex2_ftz(fmaxf(ml.x - mm, -126.f));
                    ll += ml.y * wgt;
                }
                s_w[h * kW + w] = wgt;
            }
            s_w[hq * kW + 2 * h] = mm;
            s_w[hq * kW + 2 * h + 1] = ll;
        }
        __syncthreads();
#pragma unroll 1
        for (int idx = tid; idx < hq * 128; idx += kFusedThreads) {
            const int h = idx >> 7, e = idx & 127;
            const int kvh = h / G, gg = h - kvh * G;
            const float wp = s_w[h * kW + AG::kBlocks];
            float acc = wp > 0.f ? g_o[idx] * wp : 0.f;
#pragma unroll 1
            for (int w = 0; w < nblk; ++w) {
                const float wgt = s_w[h * kW + w];
                if (wgt > 0.f) acc += part[(size_t)(w * HKV + kvh) * G * 130 + gg * 128 + e] * wgt;
            }
            g_o[idx] = acc;
        }
        if (tid < hq) g_ml[tid] = make_float2(s_w[hq * kW + 2 * tid], s_w[hq * kW + 2 * tid + 1]);
        fstamp(p, 21);
        staged = false;                                    // only the first round can have been requested early
    }
    __syncthreads();
}

// Phases 4 and 5 for everything this CTA holds.
template <int HKV, bool ATTN>
__device__ __forceinline__ void resolve_and_attend(const LayerParams& p, FusedShared& sh, unsigned char* dyn, bool& dead) {
    constexpr bool attn = ATTN;
    using AG = AttnGeom<(HKV > 0 ? HKV : 1)>;
    TailScratch& ts = tail_scratch(sh);
    // members are staged where the rotation rows and the partial outputs go later (behind the K/V rows, which
    // may already be arriving); the inline members of all records (at most kMaxGrid * kRecInline) always fit
    uint2* cand_s = reinterpret_cast<uint2*>(dyn + (attn ? AG::kCsOff : 0));
    unsigned cand_cap = attn ? (unsigned)((AG::kCsBytes + attn_part_bytes(AG::kWarpsBusy, p.group)) / 8)
                             : (unsigned)((kFusedDynSmem - 2 * kOwnCap * 4) / 8);
    const bool prepared = ATTN && ts.fast != 0 && ts.pad == 1u;
    if constexpr (ATTN) {
        if (prepared) {
            // the attention's inputs were prepared before the barrier, where the members would be staged: they go
            // behind the partial outputs instead (into the shared-memory copies of the own votes, done with here)
            cand_s = reinterpret_cast<uint2*>(dyn + early_cand_offset<HKV>(p));
            cand_cap = (unsigned)((kFusedDynSmem - early_cand_offset<HKV>(p)) / 8);
        }
    }
#pragma unroll 1
    for (int s = 0; s < sh.nseg; ++s) {
        const Resolved r = resolve_segment(p, sh, s, cand_s, cand_cap);
        emit_segment(p, sh, dyn, s, r, ts.fast != 0 && s == 0);
        fstamp(p, 16);
    }
    if constexpr (ATTN) {
        uint32_t kv_parity = 0;
        // the staged row set first (its rows are already in flight), then every other request this CTA has a part in
        const int nb = p.batch;
#pragma unroll 1
        for (int it = 0; it < 2 * nb; ++it) {
            const int pass = it >= nb ? 1 : 0, b = it - pass * nb;
            const bool is_fast = ts.fast != 0 && b == ts.fast_b;
            if ((pass == 0) != is_fast) continue;
            const StaticShare ss = static_share(p, sh, b, AG::kRows);
            const int me = share_index(p, ss);
            if (me < 0) continue;
            int st0 = me * ss.chunk, st_cnt = max(0, min(ss.total, st0 + ss.chunk) - st0);
            int own0 = 0, own_cnt = 0;
#pragma unroll 1
            for (int s = 0; s < sh.nseg; ++s)
                if (sh.seg[s].b == b) { own0 = (int)sh.seg_above[s]; own_cnt = (int)sh.seg_cnt[s]; }
            if (is_fast) {
                // staged rows: the static ones, then the possible winners (those not selected carry rank -1)
                st_cnt = ts.fast_static + ts.fast_pot;
                own_cnt = 0;
            }
            attend_rowset<HKV>(p, sh, dyn, b, sh.pbase[b] + me, st0, st_cnt, own0, own_cnt, is_fast, is_fast && prepared, kv_parity,
                               dead);
        }
    }
}

// ------------------------------------------------------------------------------------------
// phase 6: merge of the partials; one (request, head, quarter of the head dimension) per CTA at a time
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void merge_phase(const LayerParams& p, FusedShared& sh) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hq = p.hq;
    float* s_acc = reinterpret_cast<float*>(sh.hist);          // [16 warps][32]
    float* s_red = s_acc + 16 * 32;                              // [2][16]
    const int items = p.batch * hq * 4;
    fstamp(p, 22);
#pragma unroll 1
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int b = item / (hq * 4), rem = item - b * hq * 4;
        const int h = rem >> 2, qd = rem & 3;
        const int np = sh.pbase[b + 1] - sh.pbase[b];
        if (np <= 0) continue;
        const float2* ml = p.part_ml + (size_t)sh.pbase[b] * hq + h;
        const float* o = p.part_o + ((size_t)sh.pbase[b] * hq + h) * 128 + qd * 32 + lane;
        float mm = -INFINITY, ll = 0.f, acc = 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < np; c0 += 16 * 10) {
            // (max, sum) of up to 160 partials, and this warp's share of their outputs, requested together
            const int c = c0 + tid;
            float2 mine = make_float2(-INFINITY, 0.f);
            if (c < np && tid < 16 * 10) mine = __ldcg(ml + (size_t)c * hq);
            constexpr int kPer = 10;                          // partials per warp and round: one round for grids up to 160
            float xo[kPer];
#pragma unroll
            for (int u = 0; u < kPer; ++u) {
                const int cc = c0 + warp + 16 * u;
                xo[u] = cc < np ? __ldcg(o + (size_t)cc * hq * 128) : 0.f;
            }
            float m2 = mine.x;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) m2 = fmaxf(m2, __shfl_xor_sync(0xffffffffu, m2, off));
            __syncthreads();
            fstamp(p, 23);
            if (lane == 0) s_red[warp] = m2;
            __syncthreads();
            float mn = mm;
#pragma unroll
            for (int w = 0; w < 16; ++w) mn = fmaxf(mn, s_red[w]);
            const float wgt = (mine.x == -INFINITY) ? 0.f : exp2f(mine.x - mn);
            float l2 = mine.y * wgt;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) l2 += __shfl_xor_sync(0xffffffffu, l2, off);
            if (lane == 0) s_red[16 + warp] = l2;
            // weights of the partials this warp holds: partial cc belongs to thread cc - c0
            float* s_w = reinterpret_cast<float*>(sh.hist) + 1024;   // [512]
            s_w[tid] = wgt;
            __syncthreads();
            const float rescale = (mm == -INFINITY) ? 0.f : exp2f(mm - mn);
            acc *= rescale;
            ll *= rescale;
#pragma unroll
            for (int w = 0; w < 16; ++w) ll += s_red[16 + w];
#pragma unroll
            for (int u = 0; u < kPer; ++u) {
                const int cl = warp + 16 * u;
                if (c0 + cl < np) {
                    const float w = s_w[cl];
                    acc += w > 0.f ? w * xo[u] : 0.f;
                }
            }
            mm = mn;
        }
        __syncthreads();
        s_acc[warp * 32 + lane] = acc;
        __syncthreads();
        if (warp == 0) {
            float r = 0.f;
#pragma unroll
            for (int w = 0; w < 16; ++w) r += s_acc[w * 32 + lane];
            reinterpret_cast<__nv_bfloat16*>(p.out)[((size_t)b * hq + h) * 128 + qd * 32 + lane] = __float2bfloat16_rn(ll > 0.f ? r / ll : 0.f);
        }
        __syncthreads();
    }
    fstamp(p, 24);
}

}  // namespace ts
