// Token selection of one layer step as ONE persistent kernel (one CTA per SM, cooperative launch):
//
//   phase 0  per-request preparation (K/V append, query rotation, selection-cache decision)
//   phase 1  GQA query.key scoring of the candidate range [n_init, N - n_local) of every request that
//            recomputes, logits to global memory, per-CTA softmax statistics
//   phase 2  soft vote: vote[t] = sum_heads softmax_t(logit[h, :])[t], first-level histogram
//   phase 3  threshold bin of the exact top-k; winners above it counted, members of it listed
//   phase 4  remaining radix levels on the listed candidates, ordered emission of
//            init || top-k || local as logical positions and pool rows
//
// with a grid-wide barrier between phases.  Every CTA owns one contiguous range of the candidates for
// all phases, so after scoring a CTA only touches its own logits and votes plus a few small arrays
// shared through L2.
//
// Replaces, from patcher/token_retrieval.py: paged_matmul_kernel / paged_matmul (:166-261) as called
// from get_topk_tokens (:350-359); softmax + head sum (:361); max_pool1d (:366-369); topk + sort
// (:371-372); the "+ n_init" shift (:433); init || top-k || local (:436-446); the slot gather (:448);
// the cached-index reuse (:419) and cache write (:415); get_all_tokens (:329-330) for the dense
// fallback; and (phase 0) what prep.cuh lists.  The tensor-parallel exchange (:363-364) either happens
// inside the kernel after phase 2 (every CTA flags its peers and sums their votes of its own candidates
// over peer memory) or splits the kernel there: mode A ends with the raw votes, mode B starts from the
// summed votes.  A prefill chunk uses the same kernel with its fingerprint as an already rotated query.
//
// Scoring, bf16: warp 0 stages the owned part of the request's req_to_token row in shared memory a
// block at a time and issues one bulk asynchronous copy (TMA engine, mbarrier completion, L2
// evict-first) per key row of hkv*256 B into a 5-stage shared-memory ring (rows of at most four KV
// heads: eight copy warps move 16-byte cp.async pieces instead); warps 1..8 each own one
// (16-token, kv-head) unit of a stage, read it with ldmatrix and multiply it with the head group's
// queries on mma.sync m16n8k16 (tokens = M, query heads of the group = N <= 8, fp32 accumulate; bf16
// products are exact in fp32).  Rows are padded by 16 B in shared memory so the eight row addresses of
// an ldmatrix phase fall into distinct banks.  fp32 check mode (and bf16 on request) scores with plain
// loads, one warp per candidate.
//
// Top-k: radix select on the raw fp32 bit pattern (votes are >= 0, so unsigned order == value
// order); level 1 is a 2048-bin histogram of bits [30:20]; the candidates inside the threshold bin are
// resolved by further levels on (low 20 vote bits, inverted index), which makes every key distinct and
// breaks exact ties in favour of the lowest position.
//
// Logits are stored token-major, [candidate][hq], with column c = kv_head*group + j.

#include "prep.cuh"
#include "ptx.cuh"

namespace ts {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kWarps = kFusedThreads / 32;
constexpr int kBulkMinHkv = 4;        // staged scoring: bulk copies for rows of more than this many KV heads

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// CTA 0 leaves a nanosecond timestamp at every phase boundary (read back with ts_debug_read).
// (Out of line: with the stamps off, a stamp site must cost the kernel next to no instruction bytes.)
__device__ __noinline__ void stamp_slow(unsigned long long* ts, int i) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        ts[i] = t;
    }
}
// Earliest / latest CTA at the kernel's start (0), at the end of scoring (1) and at the kernel's end (2).
__device__ __noinline__ void stamp_range_slow(unsigned long long* ts, int which) {
    if (threadIdx.x != 0) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (which == 0) {
        if (blockIdx.x == 0) { ts[9] = t; ts[10] = t; ts[13] = ~0ull; ts[14] = 0ull; }
        else atomicMin(ts + 11, t);
    } else if (which == 1) {
        atomicMin(ts + 13, t);
        atomicMax(ts + 14, t);
    } else {
        atomicMax(ts + 12, t);
    }
}
__device__ __forceinline__ void stamp(const LayerParams& p, int i) {
    if (p.stamps) stamp_slow(p.phase_ts, i);
}

// Finer stamps of one ordinary CTA (CTA 1; CTA 0 also prepares the request): thread 0 at index 64 + i, a thread
// of another warp group at 96 + i.
__device__ __noinline__ void fstamp_slow(unsigned long long* ts, int i) {
    if (blockIdx.x == 1 && (threadIdx.x == 0 || threadIdx.x == 256)) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        ts[(threadIdx.x == 0 ? 64 : 96) + i] = t;
    }
}
__device__ __forceinline__ void fstamp(const LayerParams& p, int i) {
    if (p.stamps) fstamp_slow(p.phase_ts, i);
}

// ------------------------------------------------------------------------------------------
// shared state
// ------------------------------------------------------------------------------------------
constexpr int kOwnCap = 1536;          // a CTA's candidates whose votes and pool rows stay in shared memory
// Shared-memory copies of the CTA's own votes and pool rows (top of the dynamic shared memory; the ring of
// the scoring phase ends below them).
__device__ __forceinline__ float* own_votes(unsigned char* dyn) {
    return reinterpret_cast<float*>(dyn + kFusedDynSmem - 2 * kOwnCap * 4);
}
__device__ __forceinline__ int* own_slots(unsigned char* dyn) {
    return reinterpret_cast<int*>(dyn + kFusedDynSmem - kOwnCap * 4);
}
struct Seg { int b, t0, t1; };        // candidates [t0, t1) of request b owned by this CTA

struct FusedShared {
    Plan plan;
    int tile_off[kMaxBatch + 1];
    Seg seg[kMaxBatch];
    int nseg;
    PrepShared prep;
    float2 stats[16][8];              // [warp][column]
    __align__(16) float s_m[kMaxHq];   // per-head bias of the vote exponent
    unsigned long long stage_bar;      // mbarrier of the vote phase's staging copies
    unsigned hist[kHistBins];
    unsigned warp_sum[32];
    unsigned long long warp_sum64[32];
    int res_bin;
    unsigned res_above, res_cnt;
    unsigned tmp_u[4];
    int seg_b1[kMaxBatch];
    unsigned seg_above[kMaxBatch], seg_cnt[kMaxBatch];
    unsigned long long full[kScoreStages];
    unsigned long long empty[kScoreStages];
    __align__(16) int idx[2][kIdxBlock];   // (the tail's scratch overlays it and reads 16 bytes at a time)
    unsigned epoch;                    // tensor-parallel exchange: value this launch's flags carry
    int seg_off[kMaxBatch];            // start of a segment in the CTA's shared-memory copies of its votes / pool rows
    int pbase[kMaxBatch + 1];          // first attention partial of every request (see static_share)
    int own_in_smem;                   // the CTA's candidates are few enough for those copies
    unsigned tq, tr;                   // tiles per CTA: the first `tr` CTAs own tq + 1 tiles, the others tq
};

// Work tiles are dealt out in contiguous ranges, as evenly as 32-bit arithmetic makes easy: CTA c owns tiles
// [tile_lo(c), tile_lo(c + 1)).
__device__ __forceinline__ unsigned tile_lo(const FusedShared& sh, unsigned c) { return c * sh.tq + min(c, sh.tr); }
__device__ __forceinline__ int tile_owner(const FusedShared& sh, unsigned T) {
    const unsigned big = sh.tr * (sh.tq + 1u);
    return (int)(T < big ? T / (sh.tq + 1u) : sh.tr + (T - big) / sh.tq);
}

template <int HKV>
struct ScoreGeom {
    static constexpr int kTok = kScoreStageUnits / HKV;     // tokens per stage
    static constexpr int kRowBytes = HKV * 256;             // one key row (all kv heads) in the pool
    static constexpr int kRowStride = kRowBytes + 16;       // padded row in shared memory
    static constexpr int kStageBytes = kTok * kRowStride;
    static constexpr int kRowsPerLane = (kTok + 31) / 32;
    static_assert(kScoreStages * kStageBytes <= kFusedDynSmem - 2 * kOwnCap * 4, "ring must fit below the own-candidate copies");
};

// Self-resetting grid barrier (bounded).  Every CTA of the grid must call it the same number of
// times.  The word returns to its start value once all have arrived: CTA 0 adds 0x80000000-(G-1), the
// others add 1, and everyone waits for the top bit to flip.  Thread 0 keeps the top bit of the current
// generation in `gen` (read once at the start of the kernel: the bit cannot flip before this CTA has
// arrived), so arriving is a reduction that returns nothing and the wait starts at once.
__device__ __forceinline__ unsigned grid_barrier_generation(const LayerParams& p) {
    return *(volatile unsigned*)p.grid_bar & 0x80000000u;
}
// The arrival and the bounded poll, out of line (one copy for the kernel's five barriers).  Returns true
// when the wait was given up.
__device__ __noinline__ bool grid_barrier_poll(unsigned* bar, int* err, long long limit, unsigned gen, bool skip_wait,
                                                bool arrive = true) {
    if (arrive) {
        const unsigned expected = gridDim.x;
        const unsigned add = (blockIdx.x == 0) ? (0x80000000u - (expected - 1u)) : 1u;
        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(bar), "r"(add) : "memory");
    }
    if (skip_wait) return true;
    const long long t0 = clock64();
    unsigned spins = 0, v;
    while (true) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
        if (((v ^ gen) & 0x80000000u) != 0u) return false;
        if ((++spins & 255u) == 0u) {
            if (clock64() - t0 > limit) {
                set_error(err, TS_ERR_DEVICE_TIMEOUT, 10);
                return true;
            }
            if (*(volatile int*)err != 0) return true;
        }
    }
}
__device__ __forceinline__ void grid_barrier(const LayerParams& p, bool& dead, unsigned& gen) {
    __syncthreads();
    if (threadIdx.x == 0) {
        dead = grid_barrier_poll(p.grid_bar, p.err, p.wait_cycles, gen, dead);
        gen ^= 0x80000000u;
    }
    __syncthreads();
}

// The same barrier in two halves, for work that should start once this CTA's results are published but need
// not hold the other CTAs up: arrive (after a CTA barrier, thread 0), do the work, then wait.
__device__ __forceinline__ void grid_barrier_arrive(const LayerParams& p) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned add = (blockIdx.x == 0) ? (0x80000000u - (gridDim.x - 1u)) : 1u;
        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.grid_bar), "r"(add) : "memory");
    }
}
__device__ __forceinline__ void grid_barrier_wait(const LayerParams& p, bool& dead, unsigned& gen) {
    if (threadIdx.x == 0) {
        dead = grid_barrier_poll(p.grid_bar, p.err, p.wait_cycles, gen, dead, false);
        gen ^= 0x80000000u;
    }
    __syncthreads();
}

// Inclusive prefix sum over the CTA's threads (three CTA barriers inside); out of line, one copy per width.
template <typename U>
__device__ __noinline__ U block_inclusive_scan(U v, U* warp_sum) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    U inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        U t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        U w = lane < kWarps ? warp_sum[lane] : (U)0;
        U winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            U t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        warp_sum[lane] = winc - w;    // exclusive prefix of the warp totals
    }
    __syncthreads();
    U r = inc + warp_sum[warp];
    __syncthreads();
    return r;
}

// Given a 2048-bin histogram in shared memory, find the bin holding the k-th largest key (bins
// counted from the top), the number of keys in higher bins and the bin's own count.
__device__ __noinline__ void find_threshold(FusedShared& sh, unsigned k) {
    const int tid = threadIdx.x;
    constexpr int kPer = 8;            // 256 threads x 8 bins
    unsigned c[kPer];
    unsigned sum = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        c[j] = tid < kHistBins / kPer ? sh.hist[kHistBins - 1 - (tid * kPer + j)] : 0u;
        sum += c[j];
    }
    const unsigned incl = block_inclusive_scan(sum, sh.warp_sum);
    unsigned ex = incl - sum;
    if (ex < k && k <= incl) {
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            if (ex < k && k <= ex + c[j]) {
                sh.res_bin = kHistBins - 1 - (tid * kPer + j);
                sh.res_above = ex;
                sh.res_cnt = c[j];
            }
            ex += c[j];
        }
    }
    __syncthreads();
}

// The same search on a 2048-bin histogram in GLOBAL memory (one round trip, no staging copy): thread t < 256
// reads its eight consecutive bins with two 16-byte loads.
__device__ __noinline__ void find_threshold_global(FusedShared& sh, const unsigned* ghist, unsigned k) {
    const int tid = threadIdx.x;
    constexpr int kPer = 8;
    unsigned c[kPer];
    unsigned sum = 0;
    if (tid < kHistBins / kPer) {
        const uint4 lo = __ldcg(reinterpret_cast<const uint4*>(ghist + kHistBins - kPer * (tid + 1)));
        const uint4 hi = __ldcg(reinterpret_cast<const uint4*>(ghist + kHistBins - kPer * (tid + 1)) + 1);
        c[0] = hi.w; c[1] = hi.z; c[2] = hi.y; c[3] = hi.x; c[4] = lo.w; c[5] = lo.z; c[6] = lo.y; c[7] = lo.x;
    } else {
#pragma unroll
        for (int j = 0; j < kPer; ++j) c[j] = 0u;
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) sum += c[j];
    const unsigned incl = block_inclusive_scan(sum, sh.warp_sum);
    unsigned ex = incl - sum;
    if (ex < k && k <= incl) {
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            if (ex < k && k <= ex + c[j]) {
                sh.res_bin = kHistBins - 1 - (tid * kPer + j);
                sh.res_above = ex;
                sh.res_cnt = c[j];
            }
            ex += c[j];
        }
    }
    __syncthreads();
}

__device__ __forceinline__ unsigned vote_bin(float v) { return (__float_as_uint(v) >> 20) & (kHistBins - 1); }

// Count `bin` in a shared-memory histogram.  All 32 lanes of the warp call this together; lanes that hit the
// same bin elect one of them to add their number (most votes of a warp fall into a handful of bins, and
// shared-memory atomics on one address serialise).
// One shared-memory atomic per vote: merging equal bins of a warp first (match.any) measured 0.8 us slower per layer.
__device__ __forceinline__ void hist_add(unsigned* hist, unsigned bin, bool valid) {
    if (valid) atomicAdd(hist + bin, 1u);
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

// Element e of the rotated, dtype-rounded scoring query of head h (same arithmetic as prep.cuh).
template <typename T>
__device__ __forceinline__ T rotated_q(const LayerParams& p, const T* q, int h, int e) {
    if (p.q_prerot) return q[h * p.d + e];
    const int half = p.d / 2;
    const int i = e < half ? e : e - half;
    const float x1 = to_f32<T>(q[h * p.d + i]);
    const float x2 = to_f32<T>(q[h * p.d + i + half]);
    const float2 cs = p.score_cs[i];
    const float r = e < half ? __fadd_rn(__fmul_rn(x1, cs.x), __fmul_rn(-x2, cs.y))
                             : __fadd_rn(__fmul_rn(x2, cs.x), __fmul_rn(x1, cs.y));
    return from_f32<T>(r);
}

// ------------------------------------------------------------------------------------------
// Work of a layer step that the key stream does not depend on: the K/V append, the rotated scoring query
// and cache bookkeeping of the requests this CTA prepares, the window / dense / cached parts of the index
// sets it writes, and the empty softmax statistics it owes for requests it scores nothing of.  Run by a
// thread group: the whole CTA, or (staged scoring) the multiplying warps while the first key rows are in
// flight, so that the copy warps request the first key bytes as soon as the plan stands.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void emit_windows(const LayerParams& p, FusedShared& sh, const ThreadGroup& tg);

template <typename T>
__device__ __forceinline__ void side_work(const LayerParams& p, FusedShared& sh, int mode, int err0, bool ok,
                                          const ThreadGroup& tg) {
    if (mode == kModeAll || mode == kModeTpFused) {
#pragma unroll 1
        for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
            if (err0 != 0) break;
            prepare_request<T, true>(p, b, sh.prep, tg);
        }
    }
    if (!ok) return;
    if (mode != kModeTpA) emit_windows(p, sh, tg);
    // a CTA without candidates of request b still owes (-inf, 0) statistics for it
#pragma unroll 1
    for (int i = tg.tid; i < p.batch * p.hq; i += tg.nthr) {
        const int b = i / p.hq, c = i - b * p.hq;
        bool mine = false;
#pragma unroll 1
        for (int s = 0; s < sh.nseg; ++s) mine |= sh.seg[s].b == b;
        if (sh.plan.flag[b] == TS_FLAG_RECOMPUTE && !mine)
            p.partials[(size_t)b * p.part_stride + (size_t)blockIdx.x * p.hq + c] = make_float2(-INFINITY, 0.f);
    }
}

// ------------------------------------------------------------------------------------------
// phase 1, bf16: TMA ring + mma
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void producer_bar() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
__device__ __forceinline__ void cp_async_16_stream(uint32_t dst, const void* src, uint64_t pol) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "l"(pol) : "memory");
}
// This thread's arrival on the mbarrier happens when all its earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared.b64 [%0];" ::"r"(bar) : "memory");
}

// kBulk: one bulk copy (TMA engine) per key row, issued by warp 0 -- right for long rows.
// !kBulk: the eight warps that do not multiply (0 and 9..15) copy the rows in 16-byte pieces with
// cp.async, each thread arriving on the stage's mbarrier when its pieces have landed -- right for short
// rows, where the per-copy cost of the bulk engine would bound the rate.
template <typename T, int HKV, bool kBulk>
__device__ __forceinline__ void score_phase_tma(const LayerParams& p, FusedShared& sh, unsigned char* ring, bool& dead,
                                                bool side, int mode, int err0) {
    using G = ScoreGeom<HKV>;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const uint32_t ring_base = smem_u32(ring);
    const int cta = blockIdx.x;
    const int hq = p.hq, group = p.group;

    if (!kBulk && (warp == 0 || warp > 8)) {
        // ---------------- eight copying warps ----------------
        const int ptid = (warp == 0 ? 0 : warp - 8) * 32 + lane;         // 0..255
        int* slot_s = own_slots(ring);
        const unsigned char* kpool = reinterpret_cast<const unsigned char*>(p.k_pool);
        const uint64_t pol = l2_evict_first_policy();
        constexpr int kChunksPerRow = HKV * 16;                           // 16-byte pieces of a key row
        constexpr int kChunksPerThread = kScoreStageUnits * 16 / 256;     // 8
        int stage = 0;
        uint32_t phase = 0;
        for (int s = 0; s < sh.nseg; ++s) {
            const Seg sg = sh.seg[s];
            const int* row = p.rtt + (long long)sh.plan.req[sg.b] * p.rtt_stride + p.n_init;
            for (int tb0 = sg.t0; tb0 < sg.t1; tb0 += 2 * kIdxBlock) {
                const int nidx = min(2 * kIdxBlock, sg.t1 - tb0);
                int* idx = &sh.idx[0][0];
                producer_bar();                                          // the previous block's rows are all issued
                for (int i = ptid; i < nidx; i += 256) {
                    int v = __ldg(row + tb0 + i);
                    if ((unsigned long long)(long long)v >= (unsigned long long)p.pool_rows) {
                        set_error(p.err, TS_ERR_BAD_SLOT, v);
                        v = 0;
                    }
                    idx[i] = v;
                    if (sh.own_in_smem) slot_s[sh.seg_off[s] + (tb0 + i - sg.t0)] = v;
                }
                producer_bar();
                for (int t0 = 0; t0 < nidx; t0 += G::kTok) {
                    const int ntok = min(G::kTok, nidx - t0);
                    if (lane == 0) mbar_wait(smem_u32(&sh.empty[stage]), phase ^ 1u, p.err, dead, 1, p.wait_cycles);
                    __syncwarp();
                    const uint32_t dst0 = ring_base + stage * G::kStageBytes;
#pragma unroll
                    for (int j = 0; j < kChunksPerThread; ++j) {
                        const int c = ptid + 256 * j;
                        const int r = c / kChunksPerRow, o16 = c - r * kChunksPerRow;
                        if (r < ntok)
                            cp_async_16_stream(dst0 + r * G::kRowStride + o16 * 16,
                                               kpool + (size_t)idx[t0 + r] * G::kRowBytes + o16 * 16, pol);
                    }
                    cp_async_arrive_noinc(smem_u32(&sh.full[stage]));
                    if (++stage == kScoreStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");                 // nothing of ours is still in flight
        return;
    }

    if (kBulk && warp == 0) {
        // ---------------- producer ----------------
        const unsigned char* kpool = reinterpret_cast<const unsigned char*>(p.k_pool);
        const uint64_t pol = l2_evict_first_policy();
        int stage = 0;
        uint32_t phase = 0;
        uint32_t issued_mask = 0, last_parity_mask = 0;
        int buf = 0;
        for (int s = 0; s < sh.nseg; ++s) {
            const Seg sg = sh.seg[s];
            const int* row = p.rtt + (long long)sh.plan.req[sg.b] * p.rtt_stride + p.n_init;
            // index blocks: the next block's loads are in flight while this block's rows are issued
            int pre[kIdxBlock / 32];
            auto load_block = [&](int t_begin) {
#pragma unroll
                for (int j = 0; j < kIdxBlock / 32; ++j) {
                    const int t = t_begin + lane + 32 * j;
                    pre[j] = (t < sg.t1) ? __ldg(row + t) : 0;
                }
            };
            int* slot_s = own_slots(ring) + sh.seg_off[s] - sg.t0;
            auto store_block = [&](int which, int t_begin) {
#pragma unroll
                for (int j = 0; j < kIdxBlock / 32; ++j) {
                    int v = pre[j];
                    if ((unsigned long long)(long long)v >= (unsigned long long)p.pool_rows) {
                        set_error(p.err, TS_ERR_BAD_SLOT, v);
                        v = 0;
                    }
                    sh.idx[which][lane + 32 * j] = v;
                    const int t = t_begin + lane + 32 * j;
                    if (sh.own_in_smem && t < sg.t1) slot_s[t] = v;
                }
                __syncwarp();
            };
            load_block(sg.t0);
            store_block(buf, sg.t0);
            for (int tb0 = sg.t0; tb0 < sg.t1; tb0 += kIdxBlock) {
                const int tb1 = min(tb0 + kIdxBlock, sg.t1);
                const bool more = tb1 < sg.t1;
                if (more) load_block(tb1);
                for (int t0 = tb0; t0 < tb1; t0 += G::kTok) {
                    const int ntok = min(G::kTok, sg.t1 - t0);
                    mbar_wait(smem_u32(&sh.empty[stage]), phase ^ 1u, p.err, dead, 1, p.wait_cycles);
                    const uint32_t full = smem_u32(&sh.full[stage]);
                    if (lane == 0) mbar_expect_tx(full, (uint32_t)(ntok * G::kRowBytes));
                    __syncwarp();
                    const uint32_t dst0 = ring_base + stage * G::kStageBytes;
#pragma unroll
                    for (int j = 0; j < G::kRowsPerLane; ++j) {
                        const int r = lane + 32 * j;
                        if (r < ntok) {
                            const int slot = sh.idx[buf][t0 - tb0 + r];
                            bulk_row_g2s(dst0 + r * G::kRowStride, kpool + (size_t)slot * G::kRowBytes, G::kRowBytes,
                                         full, pol);
                        }
                    }
                    issued_mask |= 1u << stage;
                    last_parity_mask = (last_parity_mask & ~(1u << stage)) | (phase << stage);
                    if (++stage == kScoreStages) { stage = 0; phase ^= 1u; }
                }
                if (more) { buf ^= 1; store_block(buf, tb1); }
            }
        }
        // Do not leave the phase while copies into this CTA's shared memory may still be in flight.
        for (int s = 0; s < kScoreStages; ++s)
            if (issued_mask & (1u << s))
                mbar_wait(smem_u32(&sh.full[s]), (last_parity_mask >> s) & 1u, p.err, dead, 2, p.wait_cycles);
        return;
    }

    if (warp > 8) return;                              // only warps 1..8 multiply
    // ---------------- consumers: 8 warps, one (16-token, kv-head) unit each ----------------
    const int cw = warp - 1;
    const int ctid = tid - 32;
    // the first key rows are on their way: time for the work nothing here waits for
    if (side) side_work<T>(p, sh, mode, err0, true, ThreadGroup{ctid, 256, 1});
    const int kvh = cw % HKV;
    const int tb = cw / HKV;
    const int g = lane >> 2, t4 = lane & 3;

    // ldmatrix address of this lane inside a stage: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15)
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int lk = (lane >> 4) * 8;
    const uint32_t lane_off = (uint32_t)((tb * 16 + lrow) * G::kRowStride + kvh * 256 + lk * 2);

    int stage = 0;
    uint32_t phase = 0;
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        // B fragments: column n = g is the g-th query head paired with kv head `kvh`
        uint32_t bq[16];
        {
            const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)sg.b * hq * 128;
            const int h = (p.gqa_map == TS_GQA_MOD) ? (kvh + HKV * g) : (kvh * group + g);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    uint32_t v = 0u;
                    if (g < group) {
                        const int e = ks * 16 + 2 * t4 + 8 * u;
                        const __nv_bfloat16 lo = rotated_q<__nv_bfloat16>(p, q, h, e);
                        const __nv_bfloat16 hi = rotated_q<__nv_bfloat16>(p, q, h, e + 1);
                        v = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
                    }
                    bq[2 * ks + u] = v;
                }
            }
        }
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float* lg_base = p.logits + (size_t)sh.plan.off[sg.b] * hq + kvh * group;
        for (int t0 = sg.t0; t0 < sg.t1; t0 += G::kTok) {
            const int ntok = min(G::kTok, sg.t1 - t0);
            mbar_wait(smem_u32(&sh.full[stage]), phase, p.err, dead, 3, p.wait_cycles);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t a_base = ring_base + stage * G::kStageBytes + lane_off;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, a_base + ks * 32);
                mma_bf16_16816(acc, a, bq[2 * ks], bq[2 * ks + 1]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.empty[stage]));
            if (++stage == kScoreStages) { stage = 0; phase ^= 1u; }

            // epilogue: logits out, running (max, sum exp) per column
            const int r0 = tb * 16 + g, r1 = r0 + 8;
            const bool v0 = r0 < ntok, v1 = r1 < ntok;
            float* out0 = lg_base + (size_t)(t0 + r0) * hq;
            float* out1 = out0 + (size_t)8 * hq;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = 2 * t4 + j;
                if (c < group) {
                    const float x0 = acc[j], x1 = acc[2 + j];
                    if (v0) out0[c] = x0;
                    if (v1) out1[c] = x1;
                    const float mx = fmaxf(v0 ? x0 : -INFINITY, v1 ? x1 : -INFINITY);
                    if (mx > -INFINITY) {
                        const float mn = fmaxf(m[j], mx);
                        float sum = l[j] * exp2f((m[j] - mn) * kLog2e);
                        if (v0) sum += exp2f((x0 - mn) * kLog2e);
                        if (v1) sum += exp2f((x1 - mn) * kLog2e);
                        l[j] = sum;
                        m[j] = mn;
                    }
                }
            }
        }
        // this CTA's statistics of request sg.b: lanes -> warp -> CTA
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                float mo = __shfl_xor_sync(0xffffffffu, m[j], o);
                float lo = __shfl_xor_sync(0xffffffffu, l[j], o);
                ml_merge(m[j], l[j], mo, lo);
            }
        }
        if (g == 0) {
            sh.stats[cw][2 * t4] = make_float2(m[0], l[0]);
            sh.stats[cw][2 * t4 + 1] = make_float2(m[1], l[1]);
        }
        consumer_bar();
        if (ctid < hq) {
            const int kv = ctid / group, j = ctid - kv * group;
            float mm = -INFINITY, ll = 0.f;
            for (int w = kv; w < 8; w += HKV) ml_merge(mm, ll, sh.stats[w][j].x, sh.stats[w][j].y);
            p.partials[(size_t)sg.b * p.part_stride + (size_t)cta * hq + ctid] = make_float2(mm, ll);
        }
        consumer_bar();
    }
}

// ------------------------------------------------------------------------------------------
// phase 1, bf16, register path: every warp loads its (16-token, kv-head) units straight from the pool
// into mma A fragments with 16-byte loads (no shared-memory staging), two units in flight per warp.
// A lane's 16 bytes are eight consecutive elements of one row; the k index of an mma is only a
// summation index, so the query fragments are built in the matching permuted order:
// step s (0..3), mma m (0..1) of lane quad position t covers elements 32s + 8t + 4m + {0,1 | 2,3}.
// Used where key rows are short (few KV heads per GPU) and one bulk copy per row would be
// copy-rate bound.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_128(const void* p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}

template <int HKV>
__device__ __forceinline__ void score_phase_direct(const LayerParams& p, FusedShared& sh) {
    constexpr int WPK = kWarps / HKV;                   // warps per KV head
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int kvh = warp % HKV, wsub = warp / HKV;
    const int hq = p.hq, group = p.group;
    const unsigned char* kpool = reinterpret_cast<const unsigned char*>(p.k_pool);
    const uint64_t pol = l2_evict_first_policy();

    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        uint32_t bq[16];
        {
            const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)sg.b * hq * 128;
            const int h = (p.gqa_map == TS_GQA_MOD) ? (kvh + HKV * g) : (kvh * group + g);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                uint32_t v = 0u;
                if (g < group) {
                    const int e = 32 * (i >> 2) + 8 * t4 + 4 * ((i >> 1) & 1) + 2 * (i & 1);
                    const __nv_bfloat16 lo = rotated_q<__nv_bfloat16>(p, q, h, e);
                    const __nv_bfloat16 hi = rotated_q<__nv_bfloat16>(p, q, h, e + 1);
                    v = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
                }
                bq[i] = v;
            }
        }
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float* lg_base = p.logits + (size_t)sh.plan.off[sg.b] * hq + kvh * group;
        const int* row = p.rtt + (long long)p.req_pool_indices[sg.b] * p.rtt_stride + p.n_init;

        for (int blk0 = sg.t0; blk0 < sg.t1; blk0 += 2 * kIdxBlock) {
            const int nvalid = min(2 * kIdxBlock, sg.t1 - blk0);
            __syncthreads();
            int* idx = &sh.idx[0][0];                   // both index buffers as one block of 2*kIdxBlock
            for (int i = tid; i < nvalid; i += kFusedThreads) {
                int v = __ldg(row + blk0 + i);
                if ((unsigned long long)(long long)v >= (unsigned long long)p.pool_rows) {
                    set_error(p.err, TS_ERR_BAD_SLOT, v);
                    v = 0;
                }
                idx[i] = v;
            }
            __syncthreads();
            const int nblk = (nvalid + 15) / 16;
            auto issue = [&](int jb, uint4 (&buf)[8]) {
                const int ra = min(jb * 16 + g, nvalid - 1), rb = min(jb * 16 + g + 8, nvalid - 1);
                const unsigned char* pa = kpool + ((size_t)idx[ra] * HKV + kvh) * 256 + t4 * 16;
                const unsigned char* pb = kpool + ((size_t)idx[rb] * HKV + kvh) * 256 + t4 * 16;
#pragma unroll
                for (int st = 0; st < 4; ++st) {
                    buf[2 * st] = ldg_stream_128(pa + st * 64, pol);
                    buf[2 * st + 1] = ldg_stream_128(pb + st * 64, pol);
                }
            };
            auto consume = [&](int jb, const uint4 (&buf)[8]) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int st = 0; st < 4; ++st) {
                    const uint32_t a0[4] = {buf[2 * st].x, buf[2 * st + 1].x, buf[2 * st].y, buf[2 * st + 1].y};
                    const uint32_t a1[4] = {buf[2 * st].z, buf[2 * st + 1].z, buf[2 * st].w, buf[2 * st + 1].w};
                    mma_bf16_16816(acc, a0, bq[4 * st], bq[4 * st + 1]);
                    mma_bf16_16816(acc, a1, bq[4 * st + 2], bq[4 * st + 3]);
                }
                const int r0 = jb * 16 + g, r1 = r0 + 8;
                const bool v0 = r0 < nvalid, v1 = r1 < nvalid;
                float* out0 = lg_base + (size_t)(blk0 + r0) * hq;
                float* out1 = out0 + (size_t)8 * hq;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int c = 2 * t4 + j;
                    if (c < group) {
                        const float x0 = acc[j], x1 = acc[2 + j];
                        if (v0) out0[c] = x0;
                        if (v1) out1[c] = x1;
                        const float mx = fmaxf(v0 ? x0 : -INFINITY, v1 ? x1 : -INFINITY);
                        if (mx > -INFINITY) {
                            const float mn = fmaxf(m[j], mx);
                            float sum = l[j] * exp2f((m[j] - mn) * kLog2e);
                            if (v0) sum += exp2f((x0 - mn) * kLog2e);
                            if (v1) sum += exp2f((x1 - mn) * kLog2e);
                            l[j] = sum;
                            m[j] = mn;
                        }
                    }
                }
            };
            uint4 bufa[8], bufb[8];
            int jb = wsub;
            if (jb < nblk) issue(jb, bufa);
            while (jb < nblk) {
                if (jb + WPK < nblk) issue(jb + WPK, bufb);
                consume(jb, bufa);
                jb += WPK;
                if (jb >= nblk) break;
                if (jb + WPK < nblk) issue(jb + WPK, bufa);
                consume(jb, bufb);
                jb += WPK;
            }
        }
        // this CTA's statistics of request sg.b: lanes -> warp -> CTA
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                float mo = __shfl_xor_sync(0xffffffffu, m[j], o);
                float lo = __shfl_xor_sync(0xffffffffu, l[j], o);
                ml_merge(m[j], l[j], mo, lo);
            }
        }
        __syncthreads();
        if (g == 0) {
            sh.stats[warp][2 * t4] = make_float2(m[0], l[0]);
            sh.stats[warp][2 * t4 + 1] = make_float2(m[1], l[1]);
        }
        __syncthreads();
        if (tid < hq) {
            const int kv = tid / group, j = tid - kv * group;
            float mm = -INFINITY, ll = 0.f;
            for (int w = kv; w < kWarps; w += HKV) ml_merge(mm, ll, sh.stats[w][j].x, sh.stats[w][j].y);
            p.partials[(size_t)sg.b * p.part_stride + (size_t)blockIdx.x * hq + tid] = make_float2(mm, ll);
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// phase 1, plain loads: one warp per candidate.  q_s: rotated queries of the current request (fp32).
// ------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void score_phase_plain(const LayerParams& p, FusedShared& sh, float* q_s) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int d = p.d, hq = p.hq, hkv = p.hkv, group = p.group;
    const T* kpool = reinterpret_cast<const T*>(p.k_pool);
    float* red = reinterpret_cast<float*>(sh.hist);          // [kWarps][hq][2] scratch
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const T* q = reinterpret_cast<const T*>(p.q) + (size_t)sg.b * hq * d;
        __syncthreads();
        for (int e = tid; e < hq * d; e += kFusedThreads) q_s[e] = to_f32<T>(rotated_q<T>(p, q, e / d, e % d));
        __syncthreads();
        const int* row = p.rtt + (long long)p.req_pool_indices[sg.b] * p.rtt_stride + p.n_init;
        // lane c (and c + 32) of every warp keeps the running statistics of column c
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        for (int t = sg.t0 + warp; t < sg.t1; t += kWarps) {
            int slot = __ldg(row + t);
            if ((unsigned long long)(long long)slot >= (unsigned long long)p.pool_rows) {
                if (lane == 0) set_error(p.err, TS_ERR_BAD_SLOT, slot);
                slot = 0;
            }
            float* out = p.logits + ((size_t)sh.plan.off[sg.b] + t) * hq;
            for (int kv = 0; kv < hkv; ++kv) {
                const T* krow = kpool + ((size_t)slot * hkv + kv) * d;
                for (int j = 0; j < group; ++j) {
                    const int h = (p.gqa_map == TS_GQA_MOD) ? (kv + hkv * j) : (kv * group + j);
                    float acc = 0.f;
                    for (int e = lane; e < d; e += 32) acc = fmaf(q_s[h * d + e], to_f32<T>(krow[e]), acc);
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    const int c = kv * group + j;
                    if (lane == 0) out[c] = acc;
                    if (lane == (c & 31)) {
                        const int u = c >> 5;
                        const float mn = fmaxf(m[u], acc);
                        l[u] = l[u] * exp2f((m[u] - mn) * kLog2e) + exp2f((acc - mn) * kLog2e);
                        m[u] = mn;
                    }
                }
            }
        }
        for (int u = 0; u < 2; ++u) {
            const int c = lane + 32 * u;
            if (c < hq) { red[(warp * hq + c) * 2] = m[u]; red[(warp * hq + c) * 2 + 1] = l[u]; }
        }
        __syncthreads();
        if (tid < hq) {
            float mm = -INFINITY, ll = 0.f;
            for (int w = 0; w < kWarps; ++w) ml_merge(mm, ll, red[(w * hq + tid) * 2], red[(w * hq + tid) * 2 + 1]);
            p.partials[(size_t)sg.b * p.part_stride + (size_t)blockIdx.x * hq + tid] = make_float2(mm, ll);
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// helpers of phases 2-4: few dependent memory round trips, everything a thread needs requested at once
// ------------------------------------------------------------------------------------------
constexpr int kTokBatch = 8;          // candidates a thread holds in registers at a time

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Shared-memory stride of a staged logit row: a multiple of 16 B whose 16-byte index is odd, so that
// eight consecutive threads reading their own rows with 16-byte loads hit distinct banks.
__host__ __device__ __forceinline__ int logit_row_stride(int hq) {
    int rs = (hq * 4 + 15) / 16 * 16;
    if (((rs / 16) & 1) == 0) rs += 16;
    return rs;
}

// Votes the selection reads for candidate t: the raw vote, or the sliding maximum over
// [t - pad, t - pad + K - 1] clipped to the request (window K, padding (K-1)/2, stride 1).
__device__ __forceinline__ float sel_vote(const LayerParams& p, const float* votes, int t, int nc) {
    const int K = p.kernel_size;
    if (K <= 0) return __ldcg(votes + t);
    const int pad = (K - 1) / 2;
    const int lo = max(t - pad, 0), hi = min(t - pad + K - 1, nc - 1);
    float v = __ldcg(votes + lo);
    for (int j = lo + 1; j <= hi; ++j) v = fmaxf(v, __ldcg(votes + j));
    return v;
}

// Thread `tid` owns the consecutive candidates [own0, own1) of a segment [t0, t1).
__device__ __forceinline__ void own_range(int t0, int t1, int& own0, int& own1, int& per) {
    per = (t1 - t0 + kFusedThreads - 1) / kFusedThreads;
    own0 = min(t1, t0 + (int)threadIdx.x * per);
    own1 = min(t1, own0 + per);
}

__device__ __forceinline__ void load_vote_batch(const LayerParams& p, const float* votes, int nc, int beg, int end,
                                                float (&v)[kTokBatch]) {
#pragma unroll
    for (int i = 0; i < kTokBatch; ++i) v[i] = (beg + i < end) ? sel_vote(p, votes, beg + i, nc) : 0.f;
}

__device__ __forceinline__ void flush_hist(const LayerParams& p, FusedShared& sh, int b) {
    __syncthreads();
    unsigned* gh = p.hist + (size_t)b * kHistBins;
#pragma unroll 1
    for (int i = threadIdx.x; i < kHistBins; i += kFusedThreads) {
        const unsigned c = sh.hist[i];
        if (c) { atomicAdd(gh + i, c); sh.hist[i] = 0u; }
    }
    __syncthreads();
}

// ------------------------------------------------------------------------------------------
// phase 2: votes of the owned candidates (+ histogram).  The request's per-CTA statistics and the
// CTA's own logit rows are staged in shared memory: bulk asynchronous copies when a row is a multiple
// of 16 bytes (the rows of a CTA are one contiguous block), 4-byte asynchronous copies otherwise.
// The first block of rows is requested before the grid barrier that precedes this phase.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Flush-to-zero form: one MUFU instruction, no range fix-up around it.  Callers keep the argument above
// -126 where the result matters (see kVoteShift).
__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Vote terms are 2^(x*log2e + bias) with a non-positive exponent that can reach far below -126.  The bias
// carries +kVoteShift and the summed vote is multiplied by 2^-kVoteShift afterwards, so terms down to
// 2^-149 (the smallest fp32 denormal) are still represented exactly as the plain evaluation would.
constexpr float kVoteShift = 64.f;
constexpr float kVoteUnshift = 5.421010862427522e-20f;   // 2^-64

struct VoteGeom {
    int part_bytes, row_bytes, cap_rows;
    bool bulk;
};
__device__ __forceinline__ VoteGeom vote_geom(const LayerParams& p) {
    VoteGeom g;
    g.part_bytes = ((p.grid * p.hq + 1) & ~1) * 8;
    g.bulk = (p.hq & 3) == 0;
    g.row_bytes = g.bulk ? p.hq * 4 : logit_row_stride(p.hq);
    g.cap_rows = (kFusedDynSmem - 2 * kOwnCap * 4 - g.part_bytes) / g.row_bytes;   // below the own-candidate copies
    return g;
}

// Thread 0: request rows [r0, r1) of a segment's logits (and, with `parts`, the request's statistics).
// `armed` says the mbarrier already expects these bytes.
__device__ __forceinline__ void vote_issue(const LayerParams& p, FusedShared& sh, unsigned char* dyn, const VoteGeom& g,
                                           const Seg& sg, int r0, int r1, bool rows, bool parts, bool arm) {
    const uint32_t bar = smem_u32(&sh.stage_bar);
    const uint32_t row_total = (uint32_t)(r1 - r0) * (uint32_t)g.row_bytes;
    asm volatile("fence.proxy.async;" ::: "memory");
    if (arm) mbar_expect_tx(bar, row_total + (r0 == sg.t0 ? (uint32_t)g.part_bytes : 0u));
    if (rows) {
        const unsigned char* src =
            reinterpret_cast<const unsigned char*>(p.logits + ((size_t)sh.plan.off[sg.b] + r0) * p.hq);
        const uint32_t dst = smem_u32(dyn + g.part_bytes);
#pragma unroll 1
        for (uint32_t o = 0; o < row_total; o += 32768u)
            bulk_g2s(dst + o, src + o, min(32768u, row_total - o), bar);
    }
    if (parts)
        bulk_g2s(smem_u32(dyn), p.partials + (size_t)sg.b * p.part_stride, (uint32_t)g.part_bytes, bar);
}

// Called by all threads after the scoring phase and before the grid barrier.
__device__ __forceinline__ void vote_prefetch(const LayerParams& p, FusedShared& sh, unsigned char* dyn) {
    const VoteGeom g = vote_geom(p);
    __syncthreads();                                   // this CTA's logit stores are done
    if (g.bulk && sh.nseg > 0 && threadIdx.x == 0) {
        const Seg sg = sh.seg[0];
        vote_issue(p, sh, dyn, g, sg, sg.t0, min(sg.t1, sg.t0 + g.cap_rows), true, false, true);
    }
}

__device__ __forceinline__ void vote_phase(const LayerParams& p, FusedShared& sh, unsigned char* dyn, bool with_hist,
                                           uint32_t& stage_parity, bool& dead, float* votes_raw) {
    const int tid = threadIdx.x;
    const int hq = p.hq;
    const VoteGeom g = vote_geom(p);
    const float2* part_s = reinterpret_cast<const float2*>(dyn);
    const unsigned char* rows_s = dyn + g.part_bytes;
    const int nch = hq / 4;
    int rot_shift = 0;                                 // log2(8 / gcd(nch, 8)): see the row loop
    for (int gg = nch; (gg & 1) == 0 && rot_shift < 3; gg >>= 1) ++rot_shift;
    rot_shift = 3 - rot_shift;
    const bool pow2 = (nch & (nch - 1)) == 0;
    for (int i = tid; i < kHistBins; i += kFusedThreads) sh.hist[i] = 0u;
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const float* lg = p.logits + (size_t)sh.plan.off[sg.b] * hq;
        float* votes = votes_raw + sh.plan.off[sg.b];
        float* votes_s = own_votes(dyn) + sh.seg_off[s] - sg.t0;     // kept for the phases that follow
        for (int r0 = sg.t0; r0 < sg.t1; r0 += g.cap_rows) {
            const int r1 = min(sg.t1, r0 + g.cap_rows);
            const bool first = r0 == sg.t0;
            __syncthreads();
            if (g.bulk) {
                const bool prefetched = s == 0 && first;
                if (tid == 0) vote_issue(p, sh, dyn, g, sg, r0, r1, !prefetched, first, !prefetched);
                mbar_wait(smem_u32(&sh.stage_bar), stage_parity, p.err, dead, 4, p.wait_cycles);
                stage_parity ^= 1u;
            } else {
                if (first) {
                    const float2* src = p.partials + (size_t)sg.b * p.part_stride;
                    float2* dstp = reinterpret_cast<float2*>(dyn);
                    for (int i = tid; i < g.part_bytes / 16; i += kFusedThreads) cp_async_16(dstp + 2 * i, src + 2 * i);
                }
                for (int i = tid; i < (r1 - r0) * hq; i += kFusedThreads) {
                    const int r = i / hq, c = i - r * hq;
                    cp_async_4(dyn + g.part_bytes + (size_t)r * g.row_bytes + c * 4, lg + (size_t)(r0 + r) * hq + c);
                }
                cp_async_wait_all();
            }
            __syncthreads();
            stamp(p, 20);
            fstamp(p, 0);
            if (first) {
                // softmax statistics of the request: merge every CTA's (max, sum exp) in two levels, each
                // as a max pass followed by independent exponentials; head c then contributes
                // exp2(x*log2e + bias_c) with bias_c = -(M_c*log2e + log2 L_c)
                // Each level requests all its operands before the first is used: a loop that waits for one
                // shared-memory load per step costs more than the whole merge otherwise.
                constexpr int kMaxSlices = 16, kPerSlice = 10;
                const int nsl = min(kFusedThreads / hq, kMaxSlices);   // slices per head
                const int c = tid % hq, sl = tid / hq;
                float2* lvl = reinterpret_cast<float2*>(sh.idx);   // [nsl][hq] scratch
                if (sl < nsl) {
                    float m = -INFINITY, l = 0.f;
                    for (int i0 = sl; i0 < p.grid; i0 += nsl * kPerSlice) {   // one trip for grids up to 160 CTAs
                        float2 v[kPerSlice];
#pragma unroll
                        for (int u = 0; u < kPerSlice; ++u) {
                            const int i = i0 + u * nsl;
                            v[u] = i < p.grid ? part_s[i * hq + c] : make_float2(-INFINITY, 0.f);
                        }
                        float mn = m;
#pragma unroll
                        for (int u = 0; u < kPerSlice; ++u) mn = fmaxf(mn, v[u].x);
                        if (mn > -INFINITY) {
                            float acc = 0.f;
#pragma unroll
                            for (int u = 0; u < kPerSlice; ++u) acc += v[u].y * ex2_approx((v[u].x - mn) * kLog2e);
                            l = l * ex2_approx((m - mn) * kLog2e) + acc;
                        }
                        m = mn;
                    }
                    lvl[sl * hq + c] = make_float2(m, l);
                }
                __syncthreads();
                if (tid < hq) {
                    float2 v[kMaxSlices];
#pragma unroll
                    for (int i = 0; i < kMaxSlices; ++i)
                        v[i] = i < nsl ? lvl[i * hq + tid] : make_float2(-INFINITY, 0.f);
                    float m = -INFINITY;
#pragma unroll
                    for (int i = 0; i < kMaxSlices; ++i) m = fmaxf(m, v[i].x);
                    float l = 0.f;
#pragma unroll
                    for (int i = 0; i < kMaxSlices; ++i)
                        if (v[i].x > -INFINITY) l += v[i].y * ex2_approx((v[i].x - m) * kLog2e);
                    sh.s_m[tid] = kVoteShift - (m * kLog2e + log2f(l));
                }
                __syncthreads();
            }
            stamp(p, 21);
            fstamp(p, 1);
            if (g.bulk && nch <= 16) {
                // Rows are unpadded: every thread starts at a different 16-byte chunk so that eight
                // consecutive threads hit distinct banks (chunk counts that are not a power of two are
                // odd here and need no rotation).  A thread's rows are kFusedThreads apart, a multiple
                // of eight, so its rotation is fixed and the biases can sit in registers in that order.
                const int rot = pow2 ? ((tid >> rot_shift) & (nch - 1)) : 0;
                float4 bbr[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const int c4 = pow2 ? ((k + rot) & (nch - 1)) : k;
                    bbr[k] = k < nch ? *reinterpret_cast<const float4*>(&sh.s_m[c4 * 4]) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                const uint32_t rows_u32 = smem_u32(rows_s);
                for (int tb = r0; tb < r1; tb += kFusedThreads) {      // warp-uniform trip count
                    const int t = tb + tid;
                    const bool live = t < r1;
                    const uint32_t row = rows_u32 + (uint32_t)((live ? t : r1 - 1) - r0) * (uint32_t)g.row_bytes;
                    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        if (k < nch) {
                            const int c4 = pow2 ? ((k + rot) & (nch - 1)) : k;
                            float4 x;
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                                         : "r"(row + c4 * 16));
                            v0 += ex2_ftz(fmaf(x.x, kLog2e, bbr[k].x));
                            v1 += ex2_ftz(fmaf(x.y, kLog2e, bbr[k].y));
                            v2 += ex2_ftz(fmaf(x.z, kLog2e, bbr[k].z));
                            v3 += ex2_ftz(fmaf(x.w, kLog2e, bbr[k].w));
                        }
                    }
                    const float v = ((v0 + v1) + (v2 + v3)) * kVoteUnshift;
                    if (live) {
                        votes[t] = v;
                        if (sh.own_in_smem) votes_s[t] = v;
                    }
                    if (with_hist) hist_add(sh.hist, vote_bin(v), live);
                }
            } else {
                for (int tb = r0; tb < r1; tb += kFusedThreads) {
                    const int t = tb + tid;
                    const bool live = t < r1;
                    const float* rf = reinterpret_cast<const float*>(rows_s + (size_t)((live ? t : r1 - 1) - r0) * g.row_bytes);
                    float v = 0.f;
                    for (int c = 0; c < hq; ++c) v += ex2_ftz(fmaf(rf[c], kLog2e, sh.s_m[c]));
                    v *= kVoteUnshift;
                    if (live) {
                        votes[t] = v;
                        if (sh.own_in_smem) votes_s[t] = v;
                    }
                    if (with_hist) hist_add(sh.hist, vote_bin(v), live);
                }
            }
        }
        stamp(p, 22);
        fstamp(p, 2);
        if (with_hist) flush_hist(p, sh, sg.b);
        stamp(p, 23);
        fstamp(p, 3);
    }
}

// phase 2x (tensor parallel, fused form): every CTA tells the same-numbered CTA of every peer that
// its raw votes are written, waits for theirs, and sums the ranks' votes of its own candidates in rank
// order (so every rank gets bit-identical sums).  Replaces dist.all_reduce (token_retrieval.py:363-364).
// All ranks run the same plan, hence the same ownership.  The wait is bounded.
// The exchange for small tensor-parallel degrees: no flags, no system-scope release.  Every vote travels as an
// 8-byte (vote bits, exchange number) pair stored straight into the peers' push areas (one 8-byte store is one
// transaction, so a pair is seen whole or not at all); the receiver polls its OWN memory until a pair carries
// the current exchange number.  The areas alternate with the number's parity and the numbers only grow, so a
// pair left by an earlier exchange never matches.  Costs 8 bytes per vote and peer over NVLink instead of 4,
// which is why degrees above kPushMaxTp pull instead.
__device__ __forceinline__ void tp_exchange_push(const LayerParams& p, FusedShared& sh, unsigned char* dyn, bool with_hist,
                                                 bool& dead) {
    const int tid = threadIdx.x;
    const int tp = p.tp_size, me = p.tp_rank;
    const unsigned epoch = sh.epoch;
    const int parity = (int)(epoch & 1u);
    const size_t cap = (size_t)p.cand_capacity;
    const float* mine = p.peer_votes[parity * kMaxTp + me];
    uint2* const* push = p.peer_push + parity * kMaxTp;
    // 1. own raw votes to every peer
#pragma unroll 1
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const size_t off = (size_t)sh.plan.off[sg.b];
#pragma unroll 1
        for (int t = sg.t0 + tid; t < sg.t1; t += kFusedThreads) {
            const unsigned v = __float_as_uint(__ldcg(mine + off + t));
#pragma unroll 1
            for (int r = 0; r < tp; ++r) {
                if (r == me) continue;
                uint2* dst = push[r] + (size_t)me * cap + off + t;
                asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(v), "r"(epoch) : "memory");
            }
        }
    }
    stamp(p, 26);
#pragma unroll 1
    for (int i = tid; i < kHistBins; i += kFusedThreads) sh.hist[i] = 0u;
    __syncthreads();
    // 2. the peers' votes of the own candidates, as they arrive; summed in rank order
    const uint2* own_area = push[me];
    const long long t_begin = clock64();
    const long long peer_limit = p.wait_cycles - (p.wait_cycles >> 3);   // see tp_exchange_phase
#pragma unroll 1
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const size_t off = (size_t)sh.plan.off[sg.b];
        float* out = p.votes_final + off;
#pragma unroll 1
        for (int tb = sg.t0; tb < sg.t1; tb += kFusedThreads) {          // warp-uniform trip count
            const int t = tb + tid;
            const bool live = t < sg.t1;
            float acc = 0.f;
            if (live) {
                const float own = __ldcg(mine + off + t);
#pragma unroll 1
                for (int r = 0; r < tp; ++r) {
                    if (r == me) { acc += own; continue; }
                    const uint2* src = own_area + (size_t)r * cap + off + t;
                    uint2 v = make_uint2(0u, 0u);
                    unsigned spins = 0;
                    while (!dead) {
                        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(src) : "memory");
                        if (v.y == epoch) break;
                        if ((++spins & 63u) == 0u) {
                            if (clock64() - t_begin > peer_limit) {
                                set_error(p.err, TS_ERR_DEVICE_TIMEOUT, 30 + r);
                                dead = true;
                            } else if (*(volatile int*)p.err != 0) {
                                dead = true;
                            }
                        }
                    }
                    acc += __uint_as_float(v.x);
                }
                out[t] = acc;
                if (sh.own_in_smem) own_votes(dyn)[sh.seg_off[s] + (t - sg.t0)] = acc;
            }
            if (with_hist) hist_add(sh.hist, vote_bin(acc), live);
        }
        stamp(p, 25);
        if (with_hist) flush_hist(p, sh, sg.b);
    }
    // a wait that ran out in one thread ends the others' waits through the error word; all leave together
    dead = __syncthreads_or(dead ? 1 : 0) != 0;
}

__device__ __forceinline__ void tp_exchange_phase(const LayerParams& p, FusedShared& sh, unsigned char* dyn, bool with_hist,
                                                  bool& dead) {
    const int tid = threadIdx.x;
    const int tp = p.tp_size, me = p.tp_rank;
    __syncthreads();                                   // this CTA's raw votes are written
    // Pushing costs 8 bytes per vote and peer against 4 for pulling but saves the flag round trip and the
    // system-scope release (~4.5 us): it wins while the exchange is latency-bound.  Every CTA of every rank sees the
    // same candidate total, so all take the same branch.
    if (p.tp_push && (long long)sh.plan.off[p.batch] * (tp - 1) <= kPushMaxVotes) {
        tp_exchange_push(p, sh, dyn, with_hist, dead);
        return;
    }
    if (tid < tp && tid != me) {
        // release at system scope: the CTA's votes (ordered before this store by the barrier above) are
        // visible to the peer that observes the flag
        const unsigned epoch = sh.epoch;
        const int parity = (int)(epoch & 1u);
        unsigned* dst = p.peer_flags[tid] + ((size_t)(parity * tp + me) * kFlagPad + blockIdx.x);
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
        stamp(p, 26);
        const unsigned* src = p.peer_flags[me] + ((size_t)(parity * tp + tid) * kFlagPad + blockIdx.x);
        // a peer that stays silent is reported as such (30 + its rank): the waits for peers give up at 7/8 of the
        // limit, before a grid barrier that some CTA entered at about the same time can
        const long long t0 = clock64();
        unsigned v = 0, spins = 0;
        while (!dead) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
            if (v == epoch) break;
            if ((++spins & 63u) == 0u) {
                if (clock64() - t0 > p.wait_cycles - (p.wait_cycles >> 3)) {
                    set_error(p.err, TS_ERR_DEVICE_TIMEOUT, 30 + tid);
                    dead = true;
                } else if (*(volatile int*)p.err != 0) {
                    dead = true;
                }
            }
        }
    }
    __syncthreads();
    stamp(p, 25);
    float* const* peer_votes = p.peer_votes + (sh.epoch & 1u) * kMaxTp;
    for (int i = tid; i < kHistBins; i += kFusedThreads) sh.hist[i] = 0u;
    __syncthreads();
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const size_t off = (size_t)sh.plan.off[sg.b];
        float* out = p.votes_final + off;
        for (int tb = sg.t0; tb < sg.t1; tb += 4 * kFusedThreads) {     // warp-uniform trip count
            const int t = tb + 4 * tid;
            const bool live = t < sg.t1;
            // all ranks' pieces are requested before the first is used (one NVLink round trip), then
            // added in rank order
            float4 x[kMaxTp];
#pragma unroll
            for (int r = 0; r < kMaxTp; ++r) {
                x[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < tp && live) {
                    const float* src = peer_votes[r] + off + t;
                    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(x[r].x), "=f"(x[r].y), "=f"(x[r].z), "=f"(x[r].w)
                                 : "l"(src));
                }
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < kMaxTp; ++r) {
                if (r < tp) { acc.x += x[r].x; acc.y += x[r].y; acc.z += x[r].z; acc.w += x[r].w; }
            }
            if (live) {
                *reinterpret_cast<float4*>(out + t) = acc;
                if (sh.own_in_smem) {        // segments start on multiples of four inside a 128-aligned region
                    float* vs = own_votes(dyn) + sh.seg_off[s] + (t - sg.t0);
                    vs[0] = acc.x;
                    if (t + 1 < sg.t1) vs[1] = acc.y;
                    if (t + 2 < sg.t1) vs[2] = acc.z;
                    if (t + 3 < sg.t1) vs[3] = acc.w;
                }
            }
            if (with_hist) {
                hist_add(sh.hist, vote_bin(acc.x), live);
                hist_add(sh.hist, vote_bin(acc.y), live && t + 1 < sg.t1);
                hist_add(sh.hist, vote_bin(acc.z), live && t + 2 < sg.t1);
                hist_add(sh.hist, vote_bin(acc.w), live && t + 3 < sg.t1);
            }
        }
        if (with_hist) flush_hist(p, sh, sg.b);
    }
}

// phase 2': histogram from final votes (after a tensor-parallel sum and/or max-pool); pooled votes
// are also written out for inspection.
__device__ __forceinline__ void hist_phase(const LayerParams& p, FusedShared& sh) {
    const int tid = threadIdx.x;
    for (int i = tid; i < kHistBins; i += kFusedThreads) sh.hist[i] = 0u;
    __syncthreads();
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const int nc = sh.plan.nc[sg.b];
        const int t1 = min(sg.t1, pooled_len(nc, p.kernel_size));
        const float* votes = p.votes_final + sh.plan.off[sg.b];
        int own0, own1, per;
        own_range(sg.t0, t1, own0, own1, per);
        for (int beg = own0; beg < own1; beg += kTokBatch) {
            float v[kTokBatch];
            load_vote_batch(p, votes, nc, beg, own1, v);
#pragma unroll
            for (int i = 0; i < kTokBatch; ++i) {
                if (beg + i < own1) {
                    if (p.kernel_size > 0) p.votes_pool[sh.plan.off[sg.b] + beg + i] = v[i];
                    atomicAdd(&sh.hist[vote_bin(v[i])], 1u);
                }
            }
        }
        flush_hist(p, sh, sg.b);
    }
}

// ------------------------------------------------------------------------------------------
// phase 3: threshold bin; count the sure winners, list the threshold bin's members
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void filter_phase(const LayerParams& p, FusedShared& sh) {
    const int tid = threadIdx.x;
    // requests this CTA owns nothing of still need a zero in their per-CTA winner count
    for (int b = tid; b < p.batch; b += kFusedThreads)
        if (sh.plan.flag[b] == TS_FLAG_RECOMPUTE) p.sure_count[(size_t)b * p.grid + blockIdx.x] = 0u;
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const int nc = sh.plan.nc[sg.b];
        const int t1 = min(sg.t1, pooled_len(nc, p.kernel_size));
        const float* votes = p.votes_final + sh.plan.off[sg.b];
        uint2* cand = p.cand + sh.plan.off[sg.b];
        int own0, own1, per;
        own_range(sg.t0, t1, own0, own1, per);
        // the first batch of own votes and the request's histogram travel together
        float v0[kTokBatch];
        load_vote_batch(p, votes, nc, own0, own1, v0);
        unsigned hreg[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int bin = tid + kFusedThreads * i;
            hreg[i] = bin < kHistBins ? __ldcg(p.hist + (size_t)sg.b * kHistBins + bin) : 0u;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int bin = tid + kFusedThreads * i;
            if (bin < kHistBins) sh.hist[bin] = hreg[i];
        }
        __syncthreads();
        find_threshold(sh, (unsigned)p.top_k);
        const unsigned b1 = (unsigned)sh.res_bin;
        if (tid == 0) { sh.seg_b1[s] = sh.res_bin; sh.seg_above[s] = sh.res_above; sh.seg_cnt[s] = sh.res_cnt; }
        // pass 1: counts
        unsigned sure = 0, eq = 0;
#pragma unroll
        for (int i = 0; i < kTokBatch; ++i) {
            if (own0 + i < own1) { const unsigned bin = vote_bin(v0[i]); sure += bin > b1; eq += bin == b1; }
        }
        for (int beg = own0 + kTokBatch; beg < own1; beg += kTokBatch) {
            float v[kTokBatch];
            load_vote_batch(p, votes, nc, beg, own1, v);
#pragma unroll
            for (int i = 0; i < kTokBatch; ++i) {
                if (beg + i < own1) { const unsigned bin = vote_bin(v[i]); sure += bin > b1; eq += bin == b1; }
            }
        }
        const unsigned long long packed =
            block_inclusive_scan(((unsigned long long)sure << 32) | eq, sh.warp_sum64);
        if (tid == kFusedThreads - 1) {
            sh.tmp_u[0] = (unsigned)(packed >> 32);
            sh.tmp_u[1] = (unsigned)packed;
        }
        __syncthreads();
        if (tid == 0) {
            p.sure_count[(size_t)sg.b * p.grid + blockIdx.x] = sh.tmp_u[0];
            sh.tmp_u[2] = sh.tmp_u[1] ? atomicAdd(p.cand_count + sg.b, sh.tmp_u[1]) : 0u;
        }
        __syncthreads();
        // pass 2: append this CTA's members of the threshold bin (order inside the list is free)
        if (sh.tmp_u[1]) {
            unsigned at = sh.tmp_u[2] + (unsigned)packed - eq;
#pragma unroll
            for (int i = 0; i < kTokBatch; ++i)
                if (own0 + i < own1 && vote_bin(v0[i]) == b1)
                    cand[at++] = make_uint2((unsigned)(own0 + i), __float_as_uint(v0[i]));
            for (int beg = own0 + kTokBatch; beg < own1; beg += kTokBatch) {
                float v[kTokBatch];
                load_vote_batch(p, votes, nc, beg, own1, v);
#pragma unroll
                for (int i = 0; i < kTokBatch; ++i)
                    if (beg + i < own1 && vote_bin(v[i]) == b1)
                        cand[at++] = make_uint2((unsigned)(beg + i), __float_as_uint(v[i]));
            }
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// phase 4: remaining radix levels (every CTA for itself), ordered emission
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void emit_windows(const LayerParams& p, FusedShared& sh, const ThreadGroup& tg) {
    const int tid = tg.tid;
    const int k = p.top_k;
    // windows, dense requests and cached index sets: request b is handled by CTA grid-1 - b % grid (the
    // low-numbered CTAs prepare requests at the same time)
#pragma unroll 1
    for (int b = (int)(gridDim.x - 1 - blockIdx.x); b < p.batch; b += gridDim.x) {
        const int n = sh.plan.n[b];
        const int flag = sh.plan.flag[b];
        const int req = p.req_pool_indices[b];
        if (n < 1 || n > p.max_ctx || req < 0 || req >= p.max_reqs) {
            if (tid == 0) p.sel_count[b] = 0;
            continue;
        }
        const int* row = p.rtt + (long long)req * p.rtt_stride;
        int* out_slots = p.sel_slots + (size_t)b * p.n_sel;
        int* out_pos = p.sel_pos + (size_t)b * p.n_sel;
        if (flag == TS_FLAG_DENSE) {                       // every token, position order (:329-330)
#pragma unroll 1
            for (int i = tid; i < n; i += tg.nthr) { out_pos[i] = i; out_slots[i] = checked_slot(p, row, i); }
            if (tid == 0) p.sel_count[b] = n;
            continue;
        }
#pragma unroll 1
        for (int i = tid; i < p.n_init; i += tg.nthr) { out_pos[i] = i; out_slots[i] = checked_slot(p, row, i); }
#pragma unroll 1
        for (int i = tid; i < p.n_local; i += tg.nthr) {   // (:438-444)
            const int pos = n - p.n_local + i;
            out_pos[p.n_init + k + i] = pos;
            out_slots[p.n_init + k + i] = checked_slot(p, row, pos);
        }
        if (tid == 0) p.sel_count[b] = p.n_sel;
        if (flag == TS_FLAG_REUSE) {                       // cached positions (:419)
            const int* cache_pos = p.pos_cache + ((size_t)req * p.n_layers + p.layer) * k;
#pragma unroll 1
            for (int i = tid; i < k; i += tg.nthr) {
                const int pos = cache_pos[i];
                out_pos[p.n_init + i] = pos;
                out_slots[p.n_init + i] = checked_slot(p, row, pos);
            }
        }
    }
}

constexpr int kCandSmem = kFusedDynSmem / 8;   // threshold-bin members staged in shared memory (the idle ring)

__device__ __forceinline__ void emit_phase(const LayerParams& p, FusedShared& sh, unsigned char* dyn) {
    const int tid = threadIdx.x;
    const int k = p.top_k;
    uint2* cand_s = reinterpret_cast<uint2*>(dyn);
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const int req = p.req_pool_indices[sg.b];
        const unsigned b1 = (unsigned)sh.seg_b1[s];
        const unsigned k1 = (unsigned)k - sh.seg_above[s];       // still to take from the threshold bin
        const unsigned n_c = sh.seg_cnt[s];                      // members of the threshold bin
        const uint2* cand_g = p.cand + sh.plan.off[sg.b];
        const int nc = sh.plan.nc[sg.b];
        const int t1 = min(sg.t1, pooled_len(nc, p.kernel_size));
        const float* votes = p.votes_final + sh.plan.off[sg.b];
        int own0, own1, per;
        own_range(sg.t0, t1, own0, own1, per);

        // one round trip: first batch of own votes, lower CTAs' winner counts, the candidate list
        float v0[kTokBatch];
        load_vote_batch(p, votes, nc, own0, own1, v0);
        unsigned before = 0;
        for (int c = tid; c < (int)blockIdx.x; c += kFusedThreads) before += __ldcg(p.sure_count + (size_t)sg.b * p.grid + c);
        const bool staged = n_c <= (unsigned)kCandSmem;
        __syncthreads();
        if (staged) {
            uint2 creg[kTokBatch];
            for (unsigned i0 = 0; i0 < n_c; i0 += kFusedThreads * kTokBatch) {
#pragma unroll
                for (int u = 0; u < kTokBatch; ++u) {
                    const unsigned i = i0 + tid + kFusedThreads * u;
                    creg[u] = i < n_c ? __ldcg(cand_g + i) : make_uint2(0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < kTokBatch; ++u) {
                    const unsigned i = i0 + tid + kFusedThreads * u;
                    if (i < n_c) cand_s[i] = creg[u];
                }
            }
        }
        __syncthreads();
        auto get_cand = [&](unsigned i) -> uint2 { return staged ? cand_s[i] : __ldcg(cand_g + i); };

        // further levels on (low 20 vote bits | inverted index): 10, 10, 11, 11, 10 bits from the top
        unsigned long long prefix = 0ull, mask_above = 0ull;
        unsigned k_rem = k1, active = n_c;
        const int shifts[5] = {42, 32, 21, 10, 0};
        const unsigned widths[5] = {10, 10, 11, 11, 10};
#pragma unroll 1
        for (int lv = 0; lv < 5; ++lv) {
            if (k_rem >= active) break;                    // everything still active is taken
            __syncthreads();
            for (int i = tid; i < kHistBins; i += kFusedThreads) sh.hist[i] = 0u;
            __syncthreads();
            const unsigned long long dmask = (1ull << widths[lv]) - 1ull;
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

        // winners before this thread's candidates: lower CTAs' sure winners, winning threshold-bin
        // members below this CTA's range, own-range winners of lower threads
        for (unsigned i = tid; i < n_c; i += kFusedThreads) {
            const uint2 c = get_cand(i);
            if ((int)c.x < sg.t0 && (cand_key(c) & mask_above) >= prefix) ++before;
        }
        auto selected = [&](int t, float v) -> bool {
            const unsigned bin = vote_bin(v);
            if (bin > b1) return true;
            if (bin < b1) return false;
            return (cand_key(make_uint2((unsigned)t, __float_as_uint(v))) & mask_above) >= prefix;
        };
        unsigned mine = 0;
#pragma unroll
        for (int i = 0; i < kTokBatch; ++i) mine += (own0 + i < own1) && selected(own0 + i, v0[i]);
        for (int beg = own0 + kTokBatch; beg < own1; beg += kTokBatch) {
            float v[kTokBatch];
            load_vote_batch(p, votes, nc, beg, own1, v);
#pragma unroll
            for (int i = 0; i < kTokBatch; ++i) mine += (beg + i < own1) && selected(beg + i, v[i]);
        }
        const unsigned long long packed =
            block_inclusive_scan(((unsigned long long)before << 32) | mine, sh.warp_sum64);
        if (tid == kFusedThreads - 1) {
            sh.tmp_u[0] = (unsigned)(packed >> 32);
            sh.tmp_u[1] = (unsigned)packed;
        }
        __syncthreads();
        unsigned rank = sh.tmp_u[0] + (unsigned)packed - mine;     // rank of this thread's first winner
        const unsigned total_here = sh.tmp_u[0] + sh.tmp_u[1];

        const int* row = p.rtt + (long long)req * p.rtt_stride;
        int* out_slots = p.sel_slots + (size_t)sg.b * p.n_sel;
        int* out_pos = p.sel_pos + (size_t)sg.b * p.n_sel;
        int* cache_pos = p.pos_cache + ((size_t)req * p.n_layers + p.layer) * k;
        auto put = [&](int t) {
            if (rank < (unsigned)k) {
                const int pos = p.n_init + t;
                out_pos[p.n_init + rank] = pos;
                out_slots[p.n_init + rank] = checked_slot(p, row, pos);
                if (p.query_cache) cache_pos[rank] = pos;          // topk_indices_cache[layer] = ... (:415)
            } else {
                set_error(p.err, TS_ERR_INTERNAL, (int)rank);
            }
            ++rank;
        };
#pragma unroll
        for (int i = 0; i < kTokBatch; ++i)
            if (own0 + i < own1 && selected(own0 + i, v0[i])) put(own0 + i);
        for (int beg = own0 + kTokBatch; beg < own1; beg += kTokBatch) {
            float v[kTokBatch];
            load_vote_batch(p, votes, nc, beg, own1, v);
#pragma unroll
            for (int i = 0; i < kTokBatch; ++i)
                if (beg + i < own1 && selected(beg + i, v[i])) put(beg + i);
        }
        // the CTA owning the request's last candidates checks the total
        if (sg.t1 >= nc && tid == 0 && total_here != (unsigned)k) set_error(p.err, TS_ERR_INTERNAL, (int)total_here);
        __syncthreads();
    }
}

}  // namespace ts
#include "step_tail.cuh"
namespace ts {

// Thread 0: which candidates this CTA owns (contiguous tiles), where their shared-memory copies start, and the
// attention partials of every request.  `own_copies`: the scoring path fills the shared-memory copies.
__device__ __forceinline__ void plan_ownership(const LayerParams& p, FusedShared& sh, bool ok, bool own_copies, int attn_rows,
                                               bool attn) {
    const int tt = p.tile_tokens;
    int acc = 0;
#pragma unroll 1
    for (int b = 0; b < p.batch; ++b) { sh.tile_off[b] = acc; acc += (sh.plan.nc[b] + tt - 1) / tt; }
    sh.tile_off[p.batch] = acc;
    sh.tq = (unsigned)acc / gridDim.x;
    sh.tr = (unsigned)acc % gridDim.x;
    const int lo = (int)tile_lo(sh, blockIdx.x), hi = (int)tile_lo(sh, blockIdx.x + 1u);
    int ns = 0, own_total = 0;
#pragma unroll 1
    for (int b = 0; b < p.batch && ok; ++b) {
        const int a0 = max(lo, sh.tile_off[b]), a1 = min(hi, sh.tile_off[b + 1]);
        if (a0 < a1) {
            sh.seg[ns].b = b;
            sh.seg[ns].t0 = (a0 - sh.tile_off[b]) * tt;
            sh.seg[ns].t1 = min(sh.plan.nc[b], (a1 - sh.tile_off[b]) * tt);
            // shared-memory copies of the own votes and pool rows, when the CTA's candidates are few enough
            sh.seg_off[ns] = own_total;
            own_total += (sh.seg[ns].t1 - sh.seg[ns].t0 + 3) & ~3;
            ++ns;
        }
    }
    sh.nseg = ns;
    sh.own_in_smem = (own_copies && own_total <= kOwnCap) ? 1 : 0;
    // attention partials: one per (request, CTA that has a share of the request's rows)
    int pb = 0;
#pragma unroll 1
    for (int b = 0; b < p.batch; ++b) {
        sh.pbase[b] = pb;
        if (ok && attn) pb += static_share(p, sh, b, attn_rows).np;
    }
    sh.pbase[p.batch] = pb;
}

// ------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------
// HKV > 0: bf16 mma scoring for that many local KV heads, keys staged by bulk copies (DIRECT = false) or
// loaded straight into registers (DIRECT = true); HKV == 0: plain-load scoring.
template <typename T, int HKV, bool DIRECT>
__global__ void __launch_bounds__(kFusedThreads, 1) fused_select_kernel(const LayerParams p, const int mode) {
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ FusedShared sh;
    const int tid = threadIdx.x;
    bool dead = false;
    // Launched with programmatic serialization where the runtime accepts it together with a cooperative
    // launch: the CTAs may be placed while the previous kernel drains; nothing is read or written before it
    // has finished (no effect under a plain launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Tensor-parallel exchange inside this kernel: this CTA's exchange count picks the flag value and the
    // buffer parity (a fast rank must not overwrite votes a slow peer is still reading).  Published to the
    // CTA by the barriers that precede the first use.
    if (mode == kModeTpFused && tid == 0) {
        const unsigned e = p.cta_epoch[blockIdx.x] + 1u;
        p.cta_epoch[blockIdx.x] = e;
        sh.epoch = e;
    }

    // The attention kernels that follow are launched with programmatic serialization: let them be
    // scheduled as soon as SMs free up; they wait for this grid to finish before reading anything.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ---- phase 0 ----
    stamp(p, 0);
    stamp(p, 52 + (p.layer & 1));
    if (p.stamps) stamp_range_slow(p.phase_ts, 0);
    // The sticky error word is requested here and looked at only after the plan's own loads have been
    // issued, so that the two round trips overlap (CTAs that prepare a request need it at once).
    const int err0 = *(volatile int*)p.err;
    dead = err0 != 0;                   // a handle in error waits for nothing (its kernels do nothing either)
    unsigned bar_gen = tid == 0 ? grid_barrier_generation(p) : 0u;   // needed at the first barrier only
    const bool need_flags_barrier = p.query_cache != 0;
    // Staged scoring with the selection cache off: the flags follow from the lengths alone, so the plan is
    // built first and the per-request preparation runs on the multiplying warps while the first key rows
    // are in flight (side_work).  Otherwise the preparation (and, with the cache on, a grid barrier that
    // publishes the decisions) comes first.
    const bool side = (HKV > 0 && !DIRECT) && !need_flags_barrier && mode != kModeTpB;
    if (mode != kModeTpB && !side) {
        for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
            if (err0 != 0) break;
            if (mode == kModeAll || mode == kModeTpFused) prepare_request<T, true>(p, b, sh.prep, whole_cta());
            else if (p.query_cache) decide_request<T>(p, b, sh.prep);
        }
        if (need_flags_barrier) grid_barrier(p, dead, bar_gen);
    }
    // Flags: from the length guard alone when the selection cache is off (nothing to wait for).
    bool ok;
    if (need_flags_barrier || mode == kModeTpB) ok = build_plan<false>(p, sh.plan);
    else ok = build_plan<true>(p, sh.plan);
    ok = ok && err0 == 0;

    // ---- ownership: contiguous tile range per CTA ----
    if (tid == 0) {
        plan_ownership(p, sh, ok, HKV > 0 && !DIRECT && mode != kModeTpB, 32, false);
        mbar_init(smem_u32(&sh.stage_bar), 1);
        if (HKV > 0) {
            for (int s = 0; s < kScoreStages; ++s) {
                mbar_init(smem_u32(&sh.full[s]), (HKV > kBulkMinHkv) ? 1 : 256);
                mbar_init(smem_u32(&sh.empty[s]), 8);
            }
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t stage_parity = 0;
    // raw votes of this rank: the workspace, or (exchange inside the kernel) this rank's peer-visible buffer
    float* votes_raw = mode == kModeTpFused ? p.peer_votes[(sh.epoch & 1u) * kMaxTp + p.tp_rank] : p.votes;

    const bool pooled = p.kernel_size > 0;
    stamp(p, 1);
    // Nothing recomputes (every request reuses its cached set or attends to everything): every CTA sees
    // the same empty plan, so all of them skip the scoring phases and their barriers together.  In the
    // fused tensor-parallel form the ranks decide alike for the same reason.
    const bool nothing_to_score = sh.tile_off[p.batch] == 0;
    if (side && (nothing_to_score || !ok)) side_work<T>(p, sh, mode, err0, ok, whole_cta());
    // The parts of the index sets that do not depend on votes are written now, off the kernel's tail.
    if (!side && ok && mode != kModeTpA) emit_windows(p, sh, whole_cta());
    if (nothing_to_score) {
        stamp(p, 8);
        return;
    }
    {
        if (mode != kModeTpB) {
            // ---- phase 1: score ----
            if (ok) {
                if (!side) {
                    // a CTA without candidates of request b still owes (-inf, 0) statistics for it
                    for (int i = tid; i < p.batch * p.hq; i += kFusedThreads) {
                        const int b = i / p.hq, c = i - b * p.hq;
                        bool mine = false;
                        for (int s = 0; s < sh.nseg; ++s) mine |= sh.seg[s].b == b;
                        if (sh.plan.flag[b] == TS_FLAG_RECOMPUTE && !mine)
                            p.partials[(size_t)b * p.part_stride + (size_t)blockIdx.x * p.hq + c] = make_float2(-INFINITY, 0.f);
                    }
                }
                if constexpr (HKV > 0 && !DIRECT) score_phase_tma<T, HKV, (HKV > kBulkMinHkv)>(p, sh, ring, dead, side, mode, err0);
                else
                if constexpr (HKV > 0) score_phase_direct<HKV>(p, sh);
                else score_phase_plain<T>(p, sh, reinterpret_cast<float*>(ring));
            }
            if (ok) vote_prefetch(p, sh, ring);
            stamp(p, 2);
            if (p.stamps) stamp_range_slow(p.phase_ts, 1);
            grid_barrier(p, dead, bar_gen);
            stamp(p, 3);
            // ---- phase 2: votes ----
            if (ok) vote_phase(p, sh, ring, mode == kModeAll && !pooled, stage_parity, dead, votes_raw);
            stamp(p, 4);
            if (mode == kModeTpA) return;
            if (mode == kModeTpFused) tp_exchange_phase(p, sh, ring, ok && !pooled, dead);
            stamp(p, 24);
            if (pooled) {
                grid_barrier(p, dead, bar_gen);
                if (ok) hist_phase(p, sh);
            }
        } else {
            if (ok) hist_phase(p, sh);
        }
        grid_barrier(p, dead, bar_gen);
        stamp(p, 5);
        if (pooled) {
            // max-pooled votes: the general top-k path on the pooled vote vector; attention kernels follow
            if (ok) filter_phase(p, sh);
            stamp(p, 6);
            grid_barrier(p, dead, bar_gen);
            stamp(p, 7);
            if (ok) emit_phase(p, sh, ring);
            stamp(p, 8);
            return;
        }
        // ---- phase 3: threshold bin, records, early request of the possible winners' rows ----
        tail_init(p, sh);
        if (ok) classify_phase<HKV, false>(p, sh, ring);
        stamp(p, 6);
        grid_barrier(p, dead, bar_gen);
        stamp(p, 7);
    }
    // ---- phase 4: final set (the attention kernels follow) ----
    if (ok) resolve_and_attend<HKV, false>(p, sh, ring, dead);
    stamp(p, 8);
    if (p.stamps) stamp_range_slow(p.phase_ts, 2);
}

}  // namespace ts
#include "step_kernel.cuh"
namespace ts {

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
int fused_grid_size(int num_sms) { return num_sms; }

static bool use_mma(int dtype, unsigned flags, int hkv, int d, int group) {
    return dtype == TS_DTYPE_BF16 && !(flags & TS_CFG_PLAIN_SCORE) && d == 128 && group <= 8 &&
           (hkv == 1 || hkv == 2 || hkv == 4 || hkv == 8);
}
// The register path is an option only: staging through shared memory (bulk copies for long rows,
// cp.async pieces for short ones) measured faster at every row size (1.8x at 256-byte rows).
static bool use_direct(unsigned flags, int hkv) {
    (void)hkv;
    return (flags & TS_CFG_DIRECT_SCORE) != 0;
}

// The selection kernel can run the attention itself for the shapes its staged tensor-core scoring handles.
bool fused_attends(int dtype, unsigned flags, int hkv, int d, int group, int kernel_size, int grid) {
    return use_mma(dtype, flags, hkv, d, group) && !use_direct(flags, hkv) && kernel_size <= 0 && grid <= kMaxGrid &&
           !(flags & TS_CFG_SPLIT_ATTEND);
}
int fused_attn_rows(int hkv) { return hkv >= 4 ? 32 : 64; }

int fused_tile_tokens(int dtype, unsigned flags, int hkv, int d, int group) {
    if (!use_mma(dtype, flags, hkv, d, group) || use_direct(flags, hkv)) return 16;
    return kScoreStageUnits / hkv;
}

template <typename T, int HKV, bool DIRECT>
static cudaError_t launch_fused_t(const LayerParams& p, const Launch& l, int mode) {
    const size_t smem = kFusedDynSmem;
    static SmemConfig configured = {};
    cudaError_t e0 = ensure_dynamic_smem(fused_select_kernel<T, HKV, DIRECT>, smem, configured);
    if (e0 != cudaSuccess) return e0;
    LayerParams pp = p;
    int m = mode;
    stage_begin(l, mode == kModeTpB ? kStageSelectTpB : kStageSelect);
    // cooperative launch (all CTAs co-resident: the grid barriers need it) through the extensible
    // launch call, which queues behind the previous kernel more tightly than the dedicated call
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static bool overlap_ok = true;      // cleared the first time the runtime refuses the pair of attributes
    cfg.numAttrs = overlap_ok ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, fused_select_kernel<T, HKV, DIRECT>, pp, m);
    if (e != cudaSuccess && cfg.numAttrs == 2) {
        (void)cudaGetLastError();
        overlap_ok = false;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, fused_select_kernel<T, HKV, DIRECT>, pp, m);
    }
    stage_end(l);
    return e;
}

// The lean layer-step kernel (step_kernel.cuh): cooperative, with programmatic serialization where accepted.
template <int HKV>
static cudaError_t launch_step_t(const LayerParams& p, const Launch& l, int tp_fused) {
    const size_t smem = kFusedDynSmem;
    static SmemConfig configured = {};
    cudaError_t e0 = ensure_dynamic_smem(decode_step_kernel<HKV>, smem, configured);
    if (e0 != cudaSuccess) return e0;
    LayerParams pp = p;
    int tf = tp_fused;
    stage_begin(l, kStageSelect);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static bool overlap_ok = true;      // cleared the first time the runtime refuses the pair of attributes
    cfg.numAttrs = overlap_ok ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_step_kernel<HKV>, pp, tf);
    if (e != cudaSuccess && cfg.numAttrs == 2) {
        (void)cudaGetLastError();
        overlap_ok = false;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, decode_step_kernel<HKV>, pp, tf);
    }
    stage_end(l);
    return e;
}

cudaError_t launch_fused(const LayerParams& p, const Launch& l, int mode) {
    if (p.attn_inline && (mode == kModeAll || mode == kModeTpFused)) {
        const int tf = mode == kModeTpFused ? 1 : 0;
        switch (p.hkv) {
            case 1: return launch_step_t<1>(p, l, tf);
            case 2: return launch_step_t<2>(p, l, tf);
            case 4: return launch_step_t<4>(p, l, tf);
            default: return launch_step_t<8>(p, l, tf);
        }
    }
    if (use_mma(l.dtype, l.flags, p.hkv, p.d, p.group)) {
        const bool direct = use_direct(l.flags, p.hkv);
        switch (p.hkv) {
            case 1: return direct ? launch_fused_t<__nv_bfloat16, 1, true>(p, l, mode) : launch_fused_t<__nv_bfloat16, 1, false>(p, l, mode);
            case 2: return direct ? launch_fused_t<__nv_bfloat16, 2, true>(p, l, mode) : launch_fused_t<__nv_bfloat16, 2, false>(p, l, mode);
            case 4: return direct ? launch_fused_t<__nv_bfloat16, 4, true>(p, l, mode) : launch_fused_t<__nv_bfloat16, 4, false>(p, l, mode);
            default: return direct ? launch_fused_t<__nv_bfloat16, 8, true>(p, l, mode) : launch_fused_t<__nv_bfloat16, 8, false>(p, l, mode);
        }
    }
    if (l.dtype == TS_DTYPE_BF16) return launch_fused_t<__nv_bfloat16, 0, false>(p, l, mode);
    return launch_fused_t<float, 0, false>(p, l, mode);
}

}  // namespace ts
