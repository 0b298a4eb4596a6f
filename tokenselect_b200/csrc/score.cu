// GQA query.key scoring over the paged key pool.
//
//   logit[c, t] = sum_d q_rot[h(c), d] * Kpool[slot[n_init + t], kv(c), d]        (no scaling)
//
// Replaces paged_matmul_kernel / paged_matmul (token_retrieval.py:166-261) as called from
// get_topk_tokens (:350-359) on the candidate range [n_init, N - n_local) (:424-426).  The first
// half of the per-head softmax (:361) is fused in: every CTA also emits, per request and head, the
// running (max, sum exp) of the logits it produced.
//
// bf16 kernel: persistent CTAs, one per SM.  Warp 0 walks the request's req_to_token row and
// issues one bulk asynchronous copy (TMA engine, mbarrier completion) per key row of hkv*256 B into
// a 5-stage shared-memory ring; warps 1..8 each own one (16-token, kv-head) unit of a stage,
// read it with ldmatrix and multiply it with the head group's queries on mma.sync m16n8k16
// (tokens = M, query heads of the group = N <= 8, fp32 accumulate; bf16 products are exact in
// fp32).  Rows are padded by 16 B in shared memory so the eight row addresses of an ldmatrix
// phase fall into distinct banks.
//
// Logits are stored token-major, [candidate][hq], with column c = kv_head*group + j.
#include "common.cuh"

namespace ts {

constexpr float kLog2e = 1.4426950408889634f;

// ------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kWaitCycles, records TS_ERR_DEVICE_TIMEOUT and lets the caller
// carry on (control flow stays uniform so no barrier is left short of a participant).
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int* err, bool& dead, int where) {
    if (mbar_try_wait(bar, parity)) return;
    if (dead) return;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 1023u) == 0u) {
            if (clock64() - t0 > kWaitCycles) { set_error(err, TS_ERR_DEVICE_TIMEOUT, where); dead = true; return; }
            if (*(volatile int*)err != 0) { dead = true; return; }
        }
    }
}
// One row, global -> shared, completion counted in bytes on an mbarrier.
__device__ __forceinline__ void bulk_row_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// ------------------------------------------------------------------------------------------
// bf16 kernel
// ------------------------------------------------------------------------------------------
struct ScoreShared {
    Plan plan;
    int tile_off[kMaxBatch + 1];
    float2 stats[8][8];                 // [consumer warp][column]
    unsigned long long full[kScoreStages];
    unsigned long long empty[kScoreStages];
};

template <int HKV>
struct ScoreGeom {
    static constexpr int kTok = kScoreStageUnits / HKV;     // tokens per stage
    static constexpr int kRowBytes = HKV * 256;             // one key row (all kv heads) in the pool
    static constexpr int kRowStride = kRowBytes + 16;       // padded row in shared memory
    static constexpr int kStageBytes = kTok * kRowStride;
    static constexpr int kRowsPerLane = (kTok + 31) / 32;
};

template <int HKV>
__global__ void __launch_bounds__(kScoreThreads, 1) score_bf16_kernel(const LayerParams p) {
    using G = ScoreGeom<HKV>;
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ ScoreShared sh;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;

    if (!build_plan(p, sh.plan)) return;
    if (tid == 0) {
        int acc = 0;
        for (int b = 0; b < p.batch; ++b) { sh.tile_off[b] = acc; acc += (sh.plan.nc[b] + G::kTok - 1) / G::kTok; }
        sh.tile_off[p.batch] = acc;
        for (int s = 0; s < kScoreStages; ++s) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.empty[s]), 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int total_tiles = sh.tile_off[p.batch];
    const uint32_t ring_base = smem_u32(ring);
    bool dead = false;

    if (warp == 0) {
        // ---------------- producer: one bulk copy per key row ----------------
        const unsigned char* kpool = reinterpret_cast<const unsigned char*>(p.k_pool);
        int cur_b = 0;
        int slots[G::kRowsPerLane];
        int ntok = 0;
        auto fetch = [&](int tile, int (&out)[G::kRowsPerLane], int& out_ntok) {
            while (tile >= sh.tile_off[cur_b + 1]) ++cur_b;
            const int t0 = (tile - sh.tile_off[cur_b]) * G::kTok;
            out_ntok = min(G::kTok, sh.plan.nc[cur_b] - t0);
            const int* row = p.rtt + (long long)p.req_pool_indices[cur_b] * p.rtt_stride + p.n_init + t0;
#pragma unroll
            for (int j = 0; j < G::kRowsPerLane; ++j) {
                int r = lane + 32 * j;
                int s = 0;
                if (r < out_ntok) {
                    s = __ldg(row + r);
                    if ((unsigned long long)(long long)s >= (unsigned long long)p.pool_rows) {
                        set_error(p.err, TS_ERR_BAD_SLOT, s);
                        s = 0;
                    }
                }
                out[j] = s;
            }
        };
        int tile = blockIdx.x;
        if (tile < total_tiles) fetch(tile, slots, ntok);
        int stage = 0;
        uint32_t phase = 0;
        uint32_t issued_mask = 0, last_parity_mask = 0;
        while (tile < total_tiles) {
            const int next = tile + gridDim.x;
            int nslots[G::kRowsPerLane];
            int nntok = 0;
            if (next < total_tiles) fetch(next, nslots, nntok);   // index loads run ahead of the ring wait
            mbar_wait(smem_u32(&sh.empty[stage]), phase ^ 1u, p.err, dead, 1);
            const uint32_t full = smem_u32(&sh.full[stage]);
            if (lane == 0) mbar_expect_tx(full, (uint32_t)(ntok * G::kRowBytes));
            __syncwarp();
            const uint32_t dst0 = ring_base + stage * G::kStageBytes;
#pragma unroll
            for (int j = 0; j < G::kRowsPerLane; ++j) {
                int r = lane + 32 * j;
                if (r < ntok)
                    bulk_row_g2s(dst0 + r * G::kRowStride, kpool + (size_t)slots[j] * G::kRowBytes, G::kRowBytes, full);
            }
            issued_mask |= 1u << stage;
            last_parity_mask = (last_parity_mask & ~(1u << stage)) | (phase << stage);
            if (++stage == kScoreStages) { stage = 0; phase ^= 1u; }
            tile = next;
            ntok = nntok;
#pragma unroll
            for (int j = 0; j < G::kRowsPerLane; ++j) slots[j] = nslots[j];
        }
        // Do not leave while copies into this CTA's shared memory may still be in flight.
        for (int s = 0; s < kScoreStages; ++s)
            if (issued_mask & (1u << s))
                mbar_wait(smem_u32(&sh.full[s]), (last_parity_mask >> s) & 1u, p.err, dead, 2);
        return;
    }

    // ---------------- consumers: 8 warps, one (16-token, kv-head) unit each ----------------
    const int cw = warp - 1;
    const int ctid = tid - 32;
    const int kvh = cw % HKV;
    const int tb = cw / HKV;
    const int g = lane >> 2, t4 = lane & 3;
    const int group = p.group;
    const int hq = p.hq;
    const int cta = blockIdx.x;

    for (int i = ctid; i < p.batch * hq; i += 256) {
        int b = i / hq, c = i - b * hq;
        if (sh.plan.flag[b] == TS_FLAG_RECOMPUTE)
            p.partials[((size_t)b * p.score_grid + cta) * hq + c] = make_float2(-INFINITY, 0.f);
    }
    consumer_bar();

    // ldmatrix address of this lane inside a stage: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15)
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int lk = (lane >> 4) * 8;
    const uint32_t lane_off = (uint32_t)((tb * 16 + lrow) * G::kRowStride + kvh * 256 + lk * 2);

    uint32_t bq[16];
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int cur_b = -1;
    int scan_b = 0;

    auto flush = [&](int b) {
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
            int kv = ctid / group, j = ctid - kv * group;
            float mm = -INFINITY, ll = 0.f;
            for (int w = kv; w < 8; w += HKV) ml_merge(mm, ll, sh.stats[w][j].x, sh.stats[w][j].y);
            p.partials[((size_t)b * p.score_grid + cta) * hq + ctid] = make_float2(mm, ll);
        }
        consumer_bar();
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
    };

    int stage = 0;
    uint32_t phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        while (tile >= sh.tile_off[scan_b + 1]) ++scan_b;
        if (scan_b != cur_b) {
            if (cur_b >= 0) flush(cur_b);
            cur_b = scan_b;
            // B fragments: column n = g is the g-th query head paired with kv head `kvh`
            const __nv_bfloat16* qr = reinterpret_cast<const __nv_bfloat16*>(p.q_rot) + (size_t)cur_b * hq * 128;
            const int h = (p.gqa_map == TS_GQA_MOD) ? (kvh + HKV * g) : (kvh * group + g);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                if (g < group) {
                    bq[2 * ks] = *reinterpret_cast<const uint32_t*>(qr + h * 128 + ks * 16 + 2 * t4);
                    bq[2 * ks + 1] = *reinterpret_cast<const uint32_t*>(qr + h * 128 + ks * 16 + 2 * t4 + 8);
                } else {
                    bq[2 * ks] = 0u;
                    bq[2 * ks + 1] = 0u;
                }
            }
        }
        const int t0 = (tile - sh.tile_off[cur_b]) * G::kTok;
        const int ntok = min(G::kTok, sh.plan.nc[cur_b] - t0);

        mbar_wait(smem_u32(&sh.full[stage]), phase, p.err, dead, 3);
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
        float* out0 = p.logits + ((size_t)sh.plan.off[cur_b] + t0 + r0) * hq + kvh * group;
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
                    float s = l[j] * exp2f((m[j] - mn) * kLog2e);
                    if (v0) s += exp2f((x0 - mn) * kLog2e);
                    if (v1) s += exp2f((x1 - mn) * kLog2e);
                    l[j] = s;
                    m[j] = mn;
                }
            }
        }
    }
    if (cur_b >= 0) flush(cur_b);
}

// ------------------------------------------------------------------------------------------
// plain-load kernel: fp32 check mode (and bf16 on request); one warp per candidate token
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) score_plain_kernel(const LayerParams p) {
    __shared__ Plan plan;
    if (!build_plan(p, plan)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = blockIdx.x * 8 + warp, nw = gridDim.x * 8;
    const int d = p.d, hq = p.hq, hkv = p.hkv, group = p.group;
    const T* kpool = reinterpret_cast<const T*>(p.k_pool);
    for (int b = 0; b < p.batch; ++b) {
        const int nc = plan.nc[b];
        if (nc <= 0) continue;
        const T* qr = reinterpret_cast<const T*>(p.q_rot) + (size_t)b * hq * d;
        const int* row = p.rtt + (long long)p.req_pool_indices[b] * p.rtt_stride + p.n_init;
        for (int t = gw; t < nc; t += nw) {
            int slot = __ldg(row + t);
            if ((unsigned long long)(long long)slot >= (unsigned long long)p.pool_rows) {
                if (lane == 0) set_error(p.err, TS_ERR_BAD_SLOT, slot);
                slot = 0;
            }
            float* out = p.logits + ((size_t)plan.off[b] + t) * hq;
            for (int kv = 0; kv < hkv; ++kv) {
                const T* krow = kpool + ((size_t)slot * hkv + kv) * d;
                for (int j = 0; j < group; ++j) {
                    const int h = (p.gqa_map == TS_GQA_MOD) ? (kv + hkv * j) : (kv * group + j);
                    float s = 0.f;
                    for (int e = lane; e < d; e += 32) s = fmaf(to_f32<T>(qr[h * d + e]), to_f32<T>(krow[e]), s);
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (lane == 0) out[kv * group + j] = s;
                }
            }
        }
    }
}

// (max, sum exp) partials from stored logits; grid = (score_grid, batch).  Only after the plain kernel.
__global__ void __launch_bounds__(256) stats_from_logits_kernel(const LayerParams p) {
    __shared__ Plan plan;
    __shared__ float2 red[8];
    if (!build_plan(p, plan)) return;
    const int b = blockIdx.y;
    if (plan.flag[b] != TS_FLAG_RECOMPUTE) return;
    const int nc = plan.nc[b], hq = p.hq;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* lg = p.logits + (size_t)plan.off[b] * hq;
    for (int c = 0; c < hq; ++c) {
        float m = -INFINITY, l = 0.f;
        for (int t = blockIdx.x * 256 + threadIdx.x; t < nc; t += gridDim.x * 256) {
            float x = lg[(size_t)t * hq + c];
            float mn = fmaxf(m, x);
            l = l * exp2f((m - mn) * kLog2e) + exp2f((x - mn) * kLog2e);
            m = mn;
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            float mo = __shfl_xor_sync(0xffffffffu, m, o);
            float lo = __shfl_xor_sync(0xffffffffu, l, o);
            ml_merge(m, l, mo, lo);
        }
        if (lane == 0) red[warp] = make_float2(m, l);
        __syncthreads();
        if (threadIdx.x == 0) {
            float mm = -INFINITY, ll = 0.f;
            for (int w = 0; w < 8; ++w) ml_merge(mm, ll, red[w].x, red[w].y);
            p.partials[((size_t)b * p.score_grid + blockIdx.x) * hq + c] = make_float2(mm, ll);
        }
        __syncthreads();
    }
}

int score_grid_size(int num_sms) { return num_sms; }

size_t score_smem_bytes(int hkv) {
    switch (hkv) {
        case 1: return (size_t)kScoreStages * ScoreGeom<1>::kStageBytes;
        case 2: return (size_t)kScoreStages * ScoreGeom<2>::kStageBytes;
        case 4: return (size_t)kScoreStages * ScoreGeom<4>::kStageBytes;
        case 8: return (size_t)kScoreStages * ScoreGeom<8>::kStageBytes;
    }
    return 0;
}

template <int HKV>
static cudaError_t launch_score_bf16(const LayerParams& p, const Launch& l) {
    static bool configured = false;
    const size_t smem = (size_t)kScoreStages * ScoreGeom<HKV>::kStageBytes;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(score_bf16_kernel<HKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    score_bf16_kernel<HKV><<<p.score_grid, kScoreThreads, smem, l.stream>>>(p);
    ++*l.launch_count;
    return cudaGetLastError();
}

cudaError_t launch_score(const LayerParams& p, const Launch& l) {
    const bool fast = l.dtype == TS_DTYPE_BF16 && !(l.flags & TS_CFG_PLAIN_SCORE) && p.d == 128 && p.group <= 8 &&
                      (p.hkv == 1 || p.hkv == 2 || p.hkv == 4 || p.hkv == 8);
    if (fast) {
        switch (p.hkv) {
            case 1: return launch_score_bf16<1>(p, l);
            case 2: return launch_score_bf16<2>(p, l);
            case 4: return launch_score_bf16<4>(p, l);
            default: return launch_score_bf16<8>(p, l);
        }
    }
    if (l.dtype == TS_DTYPE_BF16) score_plain_kernel<__nv_bfloat16><<<p.score_grid, 256, 0, l.stream>>>(p);
    else score_plain_kernel<float><<<p.score_grid, 256, 0, l.stream>>>(p);
    ++*l.launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    stats_from_logits_kernel<<<dim3(p.score_grid, p.batch), 256, 0, l.stream>>>(p);
    ++*l.launch_count;
    return cudaGetLastError();
}

}  // namespace ts
