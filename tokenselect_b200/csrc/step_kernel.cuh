// The decode layer step as ONE lean kernel: K/V append, scoring, soft vote, exact top-k, sparse attention and
// the merge of its partials, for the shapes the staged tensor-core scoring handles (bf16, head_dim 128, 1/2/4/8
// KV heads per rank, no vote pooling), on one GPU or with the vote sum over ranks done inside the kernel.
// Included by fused.cu, whose general selection kernel keeps every other mode (fp32 check mode, plain and
// register scoring, the split tensor-parallel form, max-pooled votes, prefill chunks).
//
// Why a kernel of its own: every phase after the key stream runs ONCE per launch, and a phase that runs once
// costs what its instruction bytes cost to fetch (measured: a fraction of a microsecond per kilobyte, the
// instruction cache hit rate of the general kernel is ~40 %).  This kernel therefore carries no mode
// switches, keeps its cold loops rolled and calls the helpers that appear in several places out of line.
//
// Replaces patcher/token_retrieval.py:777-825 (store_kv_cache :844-854, retrieval_indices :375-449,
// get_topk_tokens :338-373 with paged_matmul :166-261, the decode attention call :815-823).
#pragma once

namespace ts {

// Votes of the CTA's candidates from its staged logit rows; compact form of vote_phase (same arithmetic).
__device__ __forceinline__ void vote_phase_lean(const LayerParams& p, FusedShared& sh, unsigned char* dyn, bool with_hist,
                                                uint32_t& stage_parity, bool& dead, float* votes_raw) {
    const int tid = threadIdx.x;
    const int hq = p.hq;
    const VoteGeom g = vote_geom(p);
    const float2* part_s = reinterpret_cast<const float2*>(dyn);
    const unsigned char* rows_s = dyn + g.part_bytes;
    const int nch = hq >> 2;
    const bool pow2 = (nch & (nch - 1)) == 0;
#pragma unroll 1
    for (int i = tid; i < kHistBins; i += kFusedThreads) sh.hist[i] = 0u;
#pragma unroll 1
    for (int s = 0; s < sh.nseg; ++s) {
        const Seg sg = sh.seg[s];
        const float* lg = p.logits + (size_t)sh.plan.off[sg.b] * hq;
        float* votes = votes_raw + sh.plan.off[sg.b];
        float* votes_s = own_votes(dyn) + sh.seg_off[s] - sg.t0;     // kept for the phases that follow
#pragma unroll 1
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
#pragma unroll 1
                    for (int i = tid; i < g.part_bytes / 16; i += kFusedThreads) cp_async_16(dstp + 2 * i, src + 2 * i);
                }
#pragma unroll 1
                for (int i = tid; i < (r1 - r0) * hq; i += kFusedThreads) {
                    const int r = i / hq, c = i - r * hq;
                    cp_async_4(dyn + g.part_bytes + (size_t)r * g.row_bytes + c * 4, lg + (size_t)(r0 + r) * hq + c);
                }
                cp_async_wait_all();
            }
            __syncthreads();
            fstamp(p, 0);
            if (first) {
                // softmax statistics of the request: every CTA's (max, sum exp); sixteen consecutive lanes share a
                // head, each takes every sixteenth CTA, a butterfly joins them; head c then contributes
                // exp2(x*log2e + bias_c) with bias_c = shift - (M_c*log2e + log2 L_c)
                auto join = [](float& m, float& l, float mo, float lo) {
                    const float mn = fmaxf(m, mo);
                    if (mn > -INFINITY)
                        l = l * ex2_ftz(fmaxf((m - mn) * kLog2e, -126.f)) + lo * ex2_ftz(fmaxf((mo - mn) * kLog2e, -126.f));
                    m = mn;
                };
#pragma unroll 1
                for (int h0 = 0; h0 < hq; h0 += kFusedThreads / 16) {
                    const int h = h0 + (tid >> 4), sl = tid & 15;
                    float m = -INFINITY, l = 0.f;
                    if (h < hq) {
#pragma unroll 1
                        for (int i = sl; i < p.grid; i += 16) {
                            const float2 v = part_s[i * hq + h];
                            join(m, l, v.x, v.y);
                        }
                    }
#pragma unroll
                    for (int o = 8; o >= 1; o >>= 1) {
                        const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, l, o);
                        join(m, l, mo, lo);
                    }
                    if (sl == 0 && h < hq) sh.s_m[h] = kVoteShift - (m * kLog2e + log2f(l));
                }
                __syncthreads();
            }
            fstamp(p, 1);
            const uint32_t rows_u32 = smem_u32(rows_s);
            const uint32_t bias_u32 = smem_u32(sh.s_m);
            // 16-byte pieces of a row: every thread starts at a different piece so that eight consecutive
            // threads hit distinct banks (piece counts that are not a power of two are odd and need no rotation)
            const int rot = pow2 ? (tid & (nch - 1)) : 0;
#pragma unroll 1
            for (int tb = r0; tb < r1; tb += kFusedThreads) {          // warp-uniform trip count
                const int t = tb + tid;
                const bool live = t < r1;
                const uint32_t row = rows_u32 + (uint32_t)((live ? t : r1 - 1) - r0) * (uint32_t)g.row_bytes;
                float v;
                if (g.bulk) {
                    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
#pragma unroll 1
                    for (int k = 0; k < nch; ++k) {
                        const int c4 = pow2 ? ((k + rot) & (nch - 1)) : k;
                        float4 x, bb;
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w) : "r"(row + c4 * 16));
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(bb.x), "=f"(bb.y), "=f"(bb.z), "=f"(bb.w) : "r"(bias_u32 + c4 * 16));
                        v0 += ex2_ftz(fmaf(x.x, kLog2e, bb.x));
                        v1 += ex2_ftz(fmaf(x.y, kLog2e, bb.y));
                        v2 += ex2_ftz(fmaf(x.z, kLog2e, bb.z));
                        v3 += ex2_ftz(fmaf(x.w, kLog2e, bb.w));
                    }
                    v = ((v0 + v1) + (v2 + v3)) * kVoteUnshift;
                } else {
                    const float* rf = reinterpret_cast<const float*>(rows_s + (size_t)((live ? t : r1 - 1) - r0) * g.row_bytes);
                    v = 0.f;
#pragma unroll 1
                    for (int c = 0; c < hq; ++c) v += ex2_ftz(fmaf(rf[c], kLog2e, sh.s_m[c]));
                    v *= kVoteUnshift;
                }
                if (live) {
                    votes[t] = v;
                    if (sh.own_in_smem) votes_s[t] = v;
                    if (with_hist) atomicAdd(&sh.hist[vote_bin(v)], 1u);
                }
            }
        }
        fstamp(p, 2);
        if (with_hist) flush_hist(p, sh, sg.b);
        fstamp(p, 3);
    }
}

template <int HKV>
__global__ void __launch_bounds__(kFusedThreads, 1) decode_step_kernel(const LayerParams p, const int tp_fused) {
    using T = __nv_bfloat16;
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ FusedShared sh;
    const int tid = threadIdx.x;
    bool dead = false;
    // Launched with programmatic serialization where the runtime accepts it: the CTAs may be placed while the
    // previous kernel drains; nothing is read or written before it has finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tp_fused && tid == 0) {
        const unsigned e = p.cta_epoch[blockIdx.x] + 1u;
        p.cta_epoch[blockIdx.x] = e;
        sh.epoch = e;
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    stamp(p, 0);
    if (p.stamps) stamp_range_slow(p.phase_ts, 0);
    const int err0 = *(volatile int*)p.err;
    dead = err0 != 0;                   // a handle in error waits for nothing (its kernels do nothing either)
    unsigned bar_gen = tid == 0 ? grid_barrier_generation(p) : 0u;
    const int mode = tp_fused ? kModeTpFused : kModeAll;
    // Selection cache off: the flags follow from the lengths alone, so the plan is built first and the
    // per-request preparation runs on the multiplying warps while the first key rows are in flight.  With the
    // cache on, the decisions come first and a grid barrier publishes them.
    const bool side = p.query_cache == 0;
    if (!side) {
#pragma unroll 1
        for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
            if (err0 != 0) break;
            prepare_request<T, true>(p, b, sh.prep, whole_cta());
        }
        grid_barrier(p, dead, bar_gen);
    }
    bool ok = side ? build_plan<true>(p, sh.plan) : build_plan<false>(p, sh.plan);
    ok = ok && err0 == 0;
    if (tid == 0) {
        plan_ownership(p, sh, ok, true, AttnGeom<HKV>::kRows, true);
        mbar_init(smem_u32(&sh.stage_bar), 1);
#pragma unroll 1
        for (int s = 0; s < kScoreStages; ++s) {
            mbar_init(smem_u32(&sh.full[s]), (HKV > kBulkMinHkv) ? 1 : 256);
            mbar_init(smem_u32(&sh.empty[s]), 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t stage_parity = 0;
    // raw votes of this rank: the workspace, or (exchange inside the kernel) this rank's peer-visible buffer
    float* votes_raw = tp_fused ? p.peer_votes[(sh.epoch & 1u) * kMaxTp + p.tp_rank] : p.votes;
    stamp(p, 1);
    const bool nothing_to_score = sh.tile_off[p.batch] == 0;
    if (side && (nothing_to_score || !ok)) side_work<T>(p, sh, mode, err0, ok, whole_cta());
    if (!side && ok) emit_windows(p, sh, whole_cta());
    if (!nothing_to_score) {
        if (ok) {
            if (!side) {
                // a CTA without candidates of request b still owes (-inf, 0) statistics for it
#pragma unroll 1
                for (int i = tid; i < p.batch * p.hq; i += kFusedThreads) {
                    const int b = i / p.hq, c = i - b * p.hq;
                    bool mine = false;
                    for (int s = 0; s < sh.nseg; ++s) mine |= sh.seg[s].b == b;
                    if (sh.plan.flag[b] == TS_FLAG_RECOMPUTE && !mine)
                        p.partials[(size_t)b * p.part_stride + (size_t)blockIdx.x * p.hq + c] = make_float2(-INFINITY, 0.f);
                }
            }
            score_phase_tma<T, HKV, (HKV > kBulkMinHkv)>(p, sh, ring, dead, side, mode, err0);
            vote_prefetch(p, sh, ring);
        }
        stamp(p, 2);
        if (p.stamps) stamp_range_slow(p.phase_ts, 1);
        grid_barrier(p, dead, bar_gen);
        stamp(p, 3);
        if (ok) vote_phase_lean(p, sh, ring, !tp_fused, stage_parity, dead, votes_raw);
        stamp(p, 4);
        if (tp_fused) tp_exchange_phase(p, sh, ring, ok, dead);
        stamp(p, 24);
        grid_barrier(p, dead, bar_gen);
        stamp(p, 5);
    }
    tail_init(p, sh);
    if (!nothing_to_score) {
        if (ok) classify_phase<HKV, true>(p, sh, ring);
        stamp(p, 6);
        grid_barrier_arrive(p);
        if (ok) {
            issue_staged_rows<HKV>(p, sh, ring);
            early_prepare<HKV>(p, sh, ring);
        }
        grid_barrier_wait(p, dead, bar_gen);
        stamp(p, 7);
    }
    if (ok) resolve_and_attend<HKV, true>(p, sh, ring, dead);
    stamp(p, 8);
    grid_barrier(p, dead, bar_gen);
    stamp(p, 15);
    if (ok) merge_phase(p, sh);
    stamp(p, 16);
    if (p.stamps) stamp_range_slow(p.phase_ts, 2);
}

}  // namespace ts
