// Sparse paged decode attention over the selected pool rows, split over the list with a
// log-sum-exp merge.
//
// Replaces the third-party paged decode call at token_retrieval.py:815-825 (planned at :802-813):
// page size 1, query rotated at position count-1, the j-th listed key at position j (rotate-half
// pairing, frequencies / rope_scale), logits * sm_scale, optional soft cap, fp32 softmax, values
// un-rotated, KV head = h / group.
//
// Split kernel: grid (chunks, batch), 16 warps.  The chunk's K and V rows and the rotation rows of its
// positions are staged in shared memory with bulk asynchronous copies (TMA engine, one mbarrier).  A
// warp works on one KV head and up to four of its query heads; eight lanes share one K/V row (lane j
// holds elements [E*j, E*j+E) of both halves of the row, i.e. both members of every rotation pair, as
// 16-byte loads), so a warp handles four listed tokens per step and a dot product needs three shuffle
// steps.  Scores of up to four steps are computed first, then one rescale and the value accumulation
// (two-pass softmax inside a group of steps).  Each group of eight lanes keeps its own softmax state;
// groups, then warps, are merged at the end.  The rotated queries sit in shared memory, laid out (like
// the rotation rows) so that the eight lanes' 16-byte loads are contiguous.
#include "ptx.cuh"

namespace ts {

constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kHeadsPerWarp = 4;
constexpr float kLog2eA = 1.4426950408889634f;

// E consecutive elements of a row as fp32.
template <typename T, int E> struct Half;
template <> struct Half<__nv_bfloat16, 8> {
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ float get(int i) const {
        const uint32_t w = i < 2 ? raw.x : i < 4 ? raw.y : i < 6 ? raw.z : raw.w;
        return __uint_as_float((i & 1) ? (w & 0xFFFF0000u) : (w << 16));
    }
};
template <> struct Half<__nv_bfloat16, 4> {
    uint2 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint2*>(p); }
    __device__ __forceinline__ float get(int i) const {
        const uint32_t w = i < 2 ? raw.x : raw.y;
        return __uint_as_float((i & 1) ? (w & 0xFFFF0000u) : (w << 16));
    }
};
template <> struct Half<float, 8> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = *reinterpret_cast<const float4*>(p);
        b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ float get(int i) const {
        return i == 0 ? a.x : i == 1 ? a.y : i == 2 ? a.z : i == 3 ? a.w : i == 4 ? b.x : i == 5 ? b.y : i == 6 ? b.z : b.w;
    }
};
template <> struct Half<float, 4> {
    float4 a;
    __device__ __forceinline__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ float get(int i) const { return i == 0 ? a.x : i == 1 ? a.y : i == 2 ? a.z : a.w; }
};

template <typename T, int E>
struct RowPair {                      // one K or V row as seen by a lane: E elements of each half
    Half<T, E> lo, hi;
    __device__ __forceinline__ void load(const T* row, int j) {
        lo.load(row + E * j);
        hi.load(row + 8 * E + E * j);
    }
};

// Shared-memory layout of the split kernel (bytes, every region 16-byte aligned).
struct AttnSmem {
    size_t q, o, ml, cs, k, v, bar, total;
};
__host__ __device__ inline AttnSmem attn_smem_layout(int hq, int hkv, int d, int ch, size_t elem) {
    AttnSmem a;
    size_t off = 0;
    a.q = off;  off += (size_t)hq * d * 4;                         // rotated queries, fp32
    a.o = off;  off += (size_t)kAttnWarps * kHeadsPerWarp * d * 4;  // per-warp partial outputs
    a.ml = off; off += (size_t)kAttnWarps * kHeadsPerWarp * 8;      // per-warp (max in base-2 units, sum)
    a.cs = off; off += (size_t)ch * (d / 2) * 8;                    // (cos, sin) rows of the chunk's positions
    a.k = off;  off += (size_t)ch * hkv * d * elem;                 // key rows of the chunk
    a.v = off;  off += (size_t)ch * hkv * d * elem;                 // value rows
    a.bar = off; off += 16;
    a.total = off;
    return a;
}

#define ATT_STAMP(i) do { if (p.stamps && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.phase_ts[(i)] = t_; } } while (0)
template <typename T, int E>
__global__ void __launch_bounds__(kAttnThreads) attend_split_kernel(const LayerParams p) {
    constexpr int D = 16 * E, HALF = 8 * E;
    constexpr int GS = kHeadsPerWarp;
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int b = blockIdx.y, chunk = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gi = lane >> 3, j = lane & 7;
    const int CH = p.attn_chunk_tokens;
    const int hkv = p.hkv, G = p.group, hq = p.hq;
    const AttnSmem lay = attn_smem_layout(hq, hkv, D, CH, sizeof(T));
    float* sm_q = reinterpret_cast<float*>(smem_raw + lay.q);
    float* sm_o = reinterpret_cast<float*>(smem_raw + lay.o);
    float2* sm_ml = reinterpret_cast<float2*>(smem_raw + lay.ml);
    const float2* sm_cs = reinterpret_cast<const float2*>(smem_raw + lay.cs);
    const T* sm_k = reinterpret_cast<const T*>(smem_raw + lay.k);
    const T* sm_v = reinterpret_cast<const T*>(smem_raw + lay.v);
    const uint32_t bar = smem_u32(smem_raw + lay.bar);

    if (tid == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    ATT_STAMP(32);
    // nothing above depends on the selection kernel; everything below does
    asm volatile("griddepcontrol.wait;" ::: "memory");
    ATT_STAMP(33);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __syncthreads();

    // one round trip: error word, sequence length, the chunk's pool rows
    const int err = *(volatile int*)p.err;
    const int n = p.seq_lens[b];
    const int base = chunk * CH;
    int my_slot = 0;
    if (warp == 0 && lane < CH) my_slot = __ldcg(p.sel_slots + (size_t)b * p.n_sel + base + lane);
    const int count = min(n, p.n_sel);                 // all tokens when the request is short (:376-378)
    if (err != 0 || base >= count) return;
    const int cnt = min(CH, count - base);
    ATT_STAMP(34);

    if (warp == 0) {
        // stage the chunk's K and V rows and rotation rows with bulk asynchronous copies
        const uint32_t row_bytes = (uint32_t)(hkv * D * sizeof(T));
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)cnt * (2u * row_bytes + (uint32_t)HALF * 8u));
        __syncwarp();
        const unsigned char* kpool = reinterpret_cast<const unsigned char*>(p.k_pool);
        const unsigned char* vpool = reinterpret_cast<const unsigned char*>(p.v_pool);
        for (int i = lane; i < cnt; i += 32) {
            int slot = (i == lane) ? my_slot : __ldcg(p.sel_slots + (size_t)b * p.n_sel + base + i);
            if ((unsigned long long)(long long)slot >= (unsigned long long)p.pool_rows) {
                set_error(p.err, TS_ERR_BAD_SLOT, slot);
                slot = 0;
            }
            bulk_g2s(smem_u32(smem_raw + lay.k) + i * row_bytes, kpool + (size_t)slot * row_bytes, row_bytes, bar);
            bulk_g2s(smem_u32(smem_raw + lay.v) + i * row_bytes, vpool + (size_t)slot * row_bytes, row_bytes, bar);
        }
        if (lane == 0)
            bulk_g2s(smem_u32(smem_raw + lay.cs), p.attn_cs_lane + (size_t)base * HALF, (uint32_t)cnt * HALF * 8u, bar);
    }
    // meanwhile: rotated query of every head at position count-1
    {
        const T* q = reinterpret_cast<const T*>(p.q) + (size_t)b * hq * D;
        const float2* cs_q = p.attn_cs + (size_t)(count - 1) * HALF;
        for (int e = tid; e < hq * HALF; e += kAttnThreads) {
            const int h = e / HALF, i = e - h * HALF;
            const float x1 = to_f32<T>(q[h * D + i]), x2 = to_f32<T>(q[h * D + i + HALF]);
            const float2 cs = cs_q[i];
            // element E*j + r of a half goes to float ((r/4)*8 + j)*4 + r%4 of that half
            const int jj = i / E, r = i - jj * E;
            const int at = ((r >> 2) * 8 + jj) * 4 + (r & 3);
            sm_q[h * D + at] = x1 * cs.x - x2 * cs.y;
            sm_q[h * D + HALF + at] = x2 * cs.x + x1 * cs.y;
        }
    }
    __syncthreads();
    ATT_STAMP(35);
    {
        bool dead = false;
        mbar_wait(bar, 0u, p.err, dead, 20, p.wait_cycles);
    }
    ATT_STAMP(36);

    const int nsg = (G + GS - 1) / GS;                 // head subgroups per KV head
    const int units = hkv * nsg;
    const int nsub = units >= kAttnWarps ? 1 : kAttnWarps / units;   // warps sharing a unit split the tokens
    const int slots_per_cta = units * nsub;            // <= 8 when units <= 8
    const float cap = p.logit_cap;

    for (int slot_id = warp; slot_id < slots_per_cta; slot_id += kAttnWarps) {
        const int unit = slot_id % units, sub = slot_id / units;
        const int kv = unit % hkv, sg = unit / hkv;
        const int g0 = sg * GS;
        const int ng = min(GS, G - g0);
        const float* qh = sm_q + (size_t)(kv * G + g0) * D;

        float m[GS], l[GS], o1[GS][E], o2[GS][E];
#pragma unroll
        for (int g = 0; g < GS; ++g) {
            m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e) { o1[g][e] = 0.f; o2[g][e] = 0.f; }
        }
        // this lane group's tokens: sub*4 + gi, then every 4*nsub; up to kSteps steps form a group whose
        // scores are all computed before the values are accumulated
        constexpr int kSteps = 1;
        const int stride = 4 * nsub;
        for (int tg0 = sub * 4; tg0 < cnt; tg0 += kSteps * stride) {
            float sc_all[kSteps][GS];
            // pass 1: scores
#pragma unroll
            for (int st = 0; st < kSteps; ++st) {
                const int tk0 = tg0 + st * stride;
#pragma unroll
                for (int g = 0; g < GS; ++g) sc_all[st][g] = -INFINITY;
                if (tk0 < cnt) {                       // warp-uniform
                    const int tk = tk0 + gi;
                    const int tkc = min(tk, cnt - 1);
                    RowPair<T, E> kf;
                    kf.load(sm_k + ((size_t)tkc * hkv + kv) * D, j);
                    float kr1[E], kr2[E];
                    const float4* cs4 = reinterpret_cast<const float4*>(sm_cs + (size_t)tkc * HALF) + j;
#pragma unroll
                    for (int e = 0; e < E; e += 2) {
                        const float4 cs = cs4[(e / 2) * 8];  // (cos, sin) of elements E*j+e and E*j+e+1
                        const float a1 = kf.lo.get(e), a2 = kf.hi.get(e);
                        const float b1 = kf.lo.get(e + 1), b2 = kf.hi.get(e + 1);
                        kr1[e] = a1 * cs.x - a2 * cs.y;
                        kr2[e] = a2 * cs.x + a1 * cs.y;
                        kr1[e + 1] = b1 * cs.z - b2 * cs.w;
                        kr2[e + 1] = b2 * cs.z + b1 * cs.w;
                    }
                    float s[GS];
#pragma unroll
                    for (int g = 0; g < GS; ++g) {
                        float a = 0.f;
                        if (g < ng) {
                            const float4* q1 = reinterpret_cast<const float4*>(qh + g * D) + j;
                            const float4* q2 = reinterpret_cast<const float4*>(qh + g * D + HALF) + j;
#pragma unroll
                            for (int e = 0; e < E; e += 4) {
                                const float4 x = q1[(e / 4) * 8], y = q2[(e / 4) * 8];
                                a += x.x * kr1[e] + x.y * kr1[e + 1] + x.z * kr1[e + 2] + x.w * kr1[e + 3];
                                a += y.x * kr2[e] + y.y * kr2[e + 1] + y.z * kr2[e + 2] + y.w * kr2[e + 3];
                            }
                        }
                        s[g] = a;
                    }
#pragma unroll
                    for (int o = 1; o <= 4; o <<= 1) {
#pragma unroll
                        for (int g = 0; g < GS; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
                    }
                    if (tk < cnt) {
#pragma unroll
                        for (int g = 0; g < GS; ++g) {
                            float x = s[g] * p.sm_scale;
                            if (cap > 0.f) x = cap * tanhf(x / cap);
                            sc_all[st][g] = x * kLog2eA;        // base-2 logits
                        }
                    }
                }
            }
            // one rescale per group of steps
            float nm[GS];
#pragma unroll
            for (int g = 0; g < GS; ++g) {
                float mx = m[g];
#pragma unroll
                for (int st = 0; st < kSteps; ++st) mx = fmaxf(mx, sc_all[st][g]);
                nm[g] = mx;
                const float sc = (mx == -INFINITY) ? 1.f : exp2f(m[g] - mx);
                l[g] *= sc;
#pragma unroll
                for (int e = 0; e < E; ++e) { o1[g][e] *= sc; o2[g][e] *= sc; }
                m[g] = mx;
            }
            // pass 2: values
#pragma unroll
            for (int st = 0; st < kSteps; ++st) {
                const int tk = tg0 + st * stride + gi;
                if (tg0 + st * stride < cnt) {           // warp-uniform
                    const int tkc = min(tk, cnt - 1);
                    RowPair<T, E> vf;
                    vf.load(sm_v + ((size_t)tkc * hkv + kv) * D, j);
                    float pe[GS];
#pragma unroll
                    for (int g = 0; g < GS; ++g) {
                        pe[g] = (sc_all[st][g] == -INFINITY) ? 0.f : exp2f(sc_all[st][g] - nm[g]);
                        l[g] += pe[g];
                    }
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        const float v1 = vf.lo.get(e), v2 = vf.hi.get(e);
#pragma unroll
                        for (int g = 0; g < GS; ++g) {
                            o1[g][e] += pe[g] * v1;
                            o2[g][e] += pe[g] * v2;
                        }
                    }
                }
            }
        }
        // merge the four lane groups (xor 8, 16)
#pragma unroll
        for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
            for (int g = 0; g < GS; ++g) {
                const float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
                const float lo = __shfl_xor_sync(0xffffffffu, l[g], off);
                const float mn = fmaxf(m[g], mo);
                const float wa = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
                const float wb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
                l[g] = l[g] * wa + lo * wb;
                m[g] = mn;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float x1 = __shfl_xor_sync(0xffffffffu, o1[g][e], off);
                    const float x2 = __shfl_xor_sync(0xffffffffu, o2[g][e], off);
                    o1[g][e] = o1[g][e] * wa + x1 * wb;
                    o2[g][e] = o2[g][e] * wa + x2 * wb;
                }
            }
        }
        if (nsub == 1) {
            // the warp owns its heads' whole chunk: write the partial straight from registers
            if (gi == 0) {
#pragma unroll
                for (int g = 0; g < GS; ++g) {
                    if (g < ng) {
                        const int h = kv * G + g0 + g;
                        float* dst = p.attn_o + (((size_t)b * p.attn_chunks + chunk) * hq + h) * D;
#pragma unroll
                        for (int e = 0; e < E; e += 4) {
                            *reinterpret_cast<float4*>(dst + E * j + e) =
                                make_float4(o1[g][e], o1[g][e + 1], o1[g][e + 2], o1[g][e + 3]);
                            *reinterpret_cast<float4*>(dst + HALF + E * j + e) =
                                make_float4(o2[g][e], o2[g][e + 1], o2[g][e + 2], o2[g][e + 3]);
                        }
                        if (j == 0) p.attn_ml[((size_t)b * p.attn_chunks + chunk) * hq + h] = make_float2(m[g], l[g]);
                    }
                }
            }
        } else if (gi == 0) {
#pragma unroll
            for (int g = 0; g < GS; ++g) {
                if (g < ng) {
                    float* dst = sm_o + ((size_t)(slot_id % kAttnWarps) * GS + g) * D;
#pragma unroll
                    for (int e = 0; e < E; ++e) { dst[E * j + e] = o1[g][e]; dst[HALF + E * j + e] = o2[g][e]; }
                    if (j == 0) sm_ml[(slot_id % kAttnWarps) * GS + g] = make_float2(m[g], l[g]);
                }
            }
        }
    }
    if (nsub == 1) { ATT_STAMP(37); ATT_STAMP(38); return; }
    __syncthreads();
    ATT_STAMP(37);
    // merge the nsub warps of each unit and write the chunk's partial
    for (int idx = tid; idx < hq * D; idx += kAttnThreads) {
        const int h = idx / D, e = idx - h * D;
        const int kv = h / G, gg = h - kv * G;
        const int unit = kv + hkv * (gg / GS), g = gg % GS;
        float mm = -INFINITY;
        for (int s = 0; s < nsub; ++s) mm = fmaxf(mm, sm_ml[(unit + s * units) * GS + g].x);
        float acc = 0.f, ll = 0.f;
        for (int s = 0; s < nsub; ++s) {
            const float2 ml = sm_ml[(unit + s * units) * GS + g];
            const float w = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - mm);
            acc += sm_o[((size_t)(unit + s * units) * GS + g) * D + e] * w;
            ll += ml.y * w;
        }
        p.attn_o[(((size_t)b * p.attn_chunks + chunk) * hq + h) * D + e] = acc;
        if (e == 0) p.attn_ml[((size_t)b * p.attn_chunks + chunk) * hq + h] = make_float2(mm, ll);
    }
    ATT_STAMP(38);
}

// ------------------------------------------------------------------------------------------
// Tensor-core split kernel (bf16, head_dim 128).  grid = (ceil(blocks / BPC), batch), BPC * HKV warps; a warp
// owns one KV head and one block of 16 listed rows.
//   S^T[heads x rows] = Q_rot . K_rot^T : A = the KV head's (<= 8) query heads, rotated, from registers;
//                        B = key rows read with ldmatrix, rotated in registers (both members of a
//                        rotation pair sit in the same lane: k-steps s and s+4);
//   O^T[d x heads]    = V^T . P^T      : A = ldmatrix.trans of the value rows, B = the softmax numerators
//                        straight from the S^T accumulators (same lane layout).
// fp32 operands (rotated Q and K, P) are split into bf16 high and low parts and multiplied in three
// (two) mma.sync so that products keep ~16 mantissa bits; V is bf16 already.  Rows, rotation tiles and
// values arrive by bulk asynchronous copies; key/value rows are padded by 16 bytes in shared memory so
// that ldmatrix phases hit distinct banks.
// ------------------------------------------------------------------------------------------

// One warp per (16-row block, KV head): BPC blocks per CTA, 32 * BPC * HKV threads.  Few rows per CTA keep
// the number of bulk copies one SM has to issue small (the copy engine issues about one per 35 ns).
template <int HKV, int BPC>
__global__ void __launch_bounds__(32 * BPC * HKV) attend_split_tc_kernel(const LayerParams p) {
    constexpr int kThreads = 32 * BPC * HKV;
    constexpr int ROWB = HKV * 256, ROWS = ROWB + 16;   // key/value row bytes in the pool / in shared memory
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* sm_k = smem_raw;
    unsigned char* sm_v = sm_k + BPC * 16 * ROWS;
    const float4* sm_cs = reinterpret_cast<const float4*>(sm_v + BPC * 16 * ROWS);   // [BPC*2 tiles][256]
    const uint32_t bar = smem_u32(sm_v + BPC * 16 * ROWS + BPC * 2 * 4096);

    const int b = blockIdx.y, blk0 = blockIdx.x * BPC;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int kv = warp % HKV, wb = warp / HKV;
    const int G = p.group, hq = p.hq;
    const int count = min(p.seq_lens[b], p.n_sel);      // inputs only: known before the selection kernel ends

    ATT_STAMP(32);
    // ---- query fragments (inputs only) ----
    uint32_t qh[8][2], ql[8][2];
    {
        const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(p.q) + ((size_t)b * hq + kv * G + min(g, G - 1)) * 128;
        const float2* csq = p.attn_cs + (size_t)max(count - 1, 0) * 64;
        uint32_t w[8][2];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int u = 0; u < 2; ++u) w[ks][u] = *reinterpret_cast<const uint32_t*>(q + 16 * ks + 8 * u + 2 * t);
#pragma unroll
        for (int s = 0; s < 4; ++s)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const float4 cs = *reinterpret_cast<const float4*>(csq + 16 * s + 8 * u + 2 * t);
                const float x1a = __uint_as_float(w[s][u] << 16), x1b = __uint_as_float(w[s][u] & 0xFFFF0000u);
                const float x2a = __uint_as_float(w[s + 4][u] << 16), x2b = __uint_as_float(w[s + 4][u] & 0xFFFF0000u);
                const bool on = g < G;
                split_bf16x2(on ? x1a * cs.x - x2a * cs.y : 0.f, on ? x1b * cs.z - x2b * cs.w : 0.f, qh[s][u], ql[s][u]);
                split_bf16x2(on ? x2a * cs.x + x1a * cs.y : 0.f, on ? x2b * cs.z + x1b * cs.w : 0.f, qh[s + 4][u], ql[s + 4][u]);
            }
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    ATT_STAMP(33);
    // nothing above depends on the selection kernel; everything below does
    asm volatile("griddepcontrol.wait;" ::: "memory");
    ATT_STAMP(34);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __syncthreads();

    const int err = *(volatile int*)p.err;
    const int base = blk0 * 16;
    if (err != 0 || base >= count) return;
    const int cnt = min(BPC * 16, count - base);
    if (warp == 0) {
        const int tiles = (cnt + 7) / 8;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)cnt * 2u * ROWB + (uint32_t)tiles * 4096u);
        __syncwarp();
        const unsigned char* kpool = reinterpret_cast<const unsigned char*>(p.k_pool);
        const unsigned char* vpool = reinterpret_cast<const unsigned char*>(p.v_pool);
        for (int i = lane; i < cnt; i += 32) {
            int slot = __ldcg(p.sel_slots + (size_t)b * p.n_sel + base + i);
            if ((unsigned long long)(long long)slot >= (unsigned long long)p.pool_rows) {
                set_error(p.err, TS_ERR_BAD_SLOT, slot);
                slot = 0;
            }
            bulk_g2s(smem_u32(sm_k) + i * ROWS, kpool + (size_t)slot * ROWB, ROWB, bar);
            bulk_g2s(smem_u32(sm_v) + i * ROWS, vpool + (size_t)slot * ROWB, ROWB, bar);
        }
        if (lane == 0)
            bulk_g2s(smem_u32(sm_cs), p.attn_cs_tile + (size_t)(base / 8) * 256, (uint32_t)tiles * 4096u, bar);
    }
    // rows past the end of the list: zeros, so that 0-weight products stay finite
    for (int i = cnt * (ROWB / 16) + tid; i < BPC * 16 * (ROWB / 16); i += kThreads) {
        const int r = i / (ROWB / 16), c = i - r * (ROWB / 16);
        *reinterpret_cast<uint4*>(sm_k + r * ROWS + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(sm_v + r * ROWS + c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    {
        bool dead = false;
        mbar_wait(bar, 0u, p.err, dead, 21, p.wait_cycles);
    }
    ATT_STAMP(35);
    const int cntb = min(16, cnt - wb * 16);             // rows of this warp's block
    if (cntb <= 0) return;

    // ---- S^T = Q_rot . K_rot^T ----
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[j][i] = 0.f;
    const int lrow = lane & 7, lsel = lane >> 3;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float4* cst = sm_cs + (size_t)((wb * 16 + 8 * j) / 8 ) * 256;
        // when a tile of eight lies wholly past the copied rotation tiles its scores are masked below
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            uint32_t r[4];
            const int doff = 16 * s + (lsel & 1) * 8 + (lsel >> 1) * 64;
            ldmatrix_x4(r, smem_u32(sm_k) + (wb * 16 + 8 * j + lrow) * ROWS + kv * 256 + doff * 2);
            uint32_t bh[2][2], bl[2][2];               // [k-step s | s+4][b0 | b1]
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const float4 cs = cst[((s * 2 + u) * 8 + g) * 4 + t];
                const float x1a = __uint_as_float(r[u] << 16), x1b = __uint_as_float(r[u] & 0xFFFF0000u);
                const float x2a = __uint_as_float(r[2 + u] << 16), x2b = __uint_as_float(r[2 + u] & 0xFFFF0000u);
                split_bf16x2(x1a * cs.x - x2a * cs.y, x1b * cs.z - x2b * cs.w, bh[0][u], bl[0][u]);
                split_bf16x2(x2a * cs.x + x1a * cs.y, x2b * cs.z + x1b * cs.w, bh[1][u], bl[1][u]);
            }
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
                const int ks = s + 4 * k2;
                const uint32_t ah[4] = {qh[ks][0], 0u, qh[ks][1], 0u};
                const uint32_t al[4] = {ql[ks][0], 0u, ql[ks][1], 0u};
                mma_bf16_16816(sc[j], ah, bh[k2][0], bh[k2][1]);
                mma_bf16_16816(sc[j], ah, bl[k2][0], bl[k2][1]);
                mma_bf16_16816(sc[j], al, bh[k2][0], bh[k2][1]);
            }
        }
    }
    ATT_STAMP(36);
    // ---- softmax over the block's rows (head = accumulator row g; a quad shares it) ----
    float x[2][2], mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            float v = sc[j][u] * p.sm_scale;
            if (p.logit_cap > 0.f) v = p.logit_cap * tanhf(v / p.logit_cap);
            v = (8 * j + 2 * t + u < cntb) ? v * kLog2eA : -INFINITY;
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
            pe[j][u] = (x[j][u] == -INFINITY) ? 0.f : exp2f(x[j][u] - mx);
            lsum += pe[j][u];
        }
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
    uint32_t ph[2], pl[2];
    split_bf16x2(pe[0][0], pe[0][1], ph[0], pl[0]);
    split_bf16x2(pe[1][0], pe[1][1], ph[1], pl[1]);

    // ---- O^T = V^T . P^T ----
    const int chunk = blk0 + wb;
    float* out_base = p.attn_o + (((size_t)b * p.attn_chunks + chunk) * hq + (size_t)kv * G) * 128;
#pragma unroll
    for (int db = 0; db < 8; ++db) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, smem_u32(sm_v) + (wb * 16 + ((lane >> 4) & 1) * 8 + lrow) * ROWS + kv * 256 +
                                 (16 * db + ((lane >> 3) & 1) * 8) * 2);
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        mma_bf16_16816(o, a, ph[0], ph[1]);
        mma_bf16_16816(o, a, pl[0], pl[1]);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int hh = 2 * t + u;
            if (hh < G) {
                out_base[(size_t)hh * 128 + 16 * db + g] = o[u];
                out_base[(size_t)hh * 128 + 16 * db + g + 8] = o[2 + u];
            }
        }
    }
    if (t == 0 && g < G) p.attn_ml[((size_t)b * p.attn_chunks + chunk) * hq + kv * G + g] = make_float2(mx, lsum);
    ATT_STAMP(37);
}

// grid = (hq, batch), block = 512: warp w takes chunks w, w+16, ...; lane i takes elements
// [VEC*i, VEC*i + VEC).  The partial outputs are requested before the weights are known.
constexpr int kMergeThreads = 512;
constexpr int kMergeBatch = 12;
template <typename T, int VEC>
__global__ void __launch_bounds__(kMergeThreads) attend_merge_kernel(const LayerParams p) {
    constexpr int D = 32 * VEC;
    constexpr int NW = kMergeThreads / 32;
    __shared__ float s_w[kMergeThreads];
    __shared__ float s_acc[NW][D];
    __shared__ float s_red[2 * NW];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next layer's first kernel may be placed
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hq = p.hq;
    ATT_STAMP(48 + 2 * (p.layer & 1));
    const int err = *(volatile int*)p.err;
    const int count = min(p.seq_lens[b], p.n_sel);
    if (err != 0 || count < 1) return;
    const int chunks = (count + p.attn_chunk_tokens - 1) / p.attn_chunk_tokens;
    const float2* ml = p.attn_ml + (size_t)b * p.attn_chunks * hq + h;
    const float* o = p.attn_o + ((size_t)b * p.attn_chunks * hq + h) * D + VEC * lane;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
    float mm_run = -INFINITY, ll_run = 0.f;            // running (max, sum) over chunk rounds
    for (int c0 = 0; c0 < chunks; c0 += kMergeThreads) {
        // the (max, sum) of up to 512 chunks and this warp's partial outputs travel together
        const int c = c0 + tid;
        float2 mine = make_float2(-INFINITY, 0.f);
        if (c < chunks) mine = __ldcg(ml + (size_t)c * hq);
        float xo[kMergeBatch][VEC];
        const int nround = min(kMergeThreads, chunks - c0);
#pragma unroll
        for (int u = 0; u < kMergeBatch; ++u) {
            const int cc = warp + NW * u;
#pragma unroll
            for (int v = 0; v < VEC; ++v) xo[u][v] = 0.f;
            if (cc < nround) {
                const float* src = o + (size_t)(c0 + cc) * hq * D;
                if (VEC == 4) {
                    const float4 x = __ldcg(reinterpret_cast<const float4*>(src));
                    xo[u][0] = x.x; xo[u][1] = x.y; xo[u][VEC - 2] = x.z; xo[u][VEC - 1] = x.w;
                } else {
                    const float2 x = __ldcg(reinterpret_cast<const float2*>(src));
                    xo[u][0] = x.x; xo[u][VEC - 1] = x.y;
                }
            }
        }
        float mm = mine.x;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
        if (lane == 0) s_red[warp] = mm;
        __syncthreads();
        mm = mm_run;
#pragma unroll
        for (int w = 0; w < NW; ++w) mm = fmaxf(mm, s_red[w]);
        const float wgt = (mine.x == -INFINITY) ? 0.f : exp2f(mine.x - mm);
        s_w[tid] = wgt;
        float ll = mine.y * wgt;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, off);
        if (lane == 0) s_red[NW + warp] = ll;
        __syncthreads();
        const float rescale = (mm_run == -INFINITY) ? 0.f : exp2f(mm_run - mm);
        ll = ll_run * rescale;
#pragma unroll
        for (int w = 0; w < NW; ++w) ll += s_red[NW + w];
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] *= rescale;
#pragma unroll
        for (int u = 0; u < kMergeBatch; ++u) {
            const int cc = warp + NW * u;
            if (cc < nround) {
                const float w = s_w[cc];
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[v] += w * xo[u][v];
            }
        }
        // chunks of this round beyond the register batch (only with very long lists)
        for (int cc = warp + NW * kMergeBatch; cc < nround; cc += NW) {
            const float w = s_w[cc];
            const float* src = o + (size_t)(c0 + cc) * hq * D;
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] += w * __ldcg(src + v);
        }
        mm_run = mm;
        ll_run = ll;
        __syncthreads();
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) s_acc[warp][VEC * lane + v] = acc[v];
    __syncthreads();
    for (int e = tid; e < D; e += kMergeThreads) {
        float r = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) r += s_acc[w][e];
        reinterpret_cast<T*>(p.out)[((size_t)b * hq + h) * D + e] = from_f32<T>(r / ll_run);
    }
    ATT_STAMP(49 + 2 * (p.layer & 1));
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor
// drains; it waits (griddepcontrol.wait) before touching anything the predecessor wrote.
template <typename... Args>
static cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <typename T, int E>
static cudaError_t launch_attend_t(const LayerParams& p, const Launch& l) {
    constexpr int D = 16 * E;
    const size_t smem = attn_smem_layout(p.hq, p.hkv, D, p.attn_chunk_tokens, sizeof(T)).total;
    static SmemConfig configured = {};
    cudaError_t e = ensure_dynamic_smem(attend_split_kernel<T, E>, smem, configured);
    if (e != cudaSuccess) return e;
    stage_begin(l, kStageAttendSplit);
    e = launch_pdl(attend_split_kernel<T, E>, dim3(p.attn_chunks, p.batch), dim3(kAttnThreads), smem,
                               l.stream, p);
    stage_end(l);
    if (e != cudaSuccess) return e;
    stage_begin(l, kStageAttendMerge);
    e = launch_pdl(attend_merge_kernel<T, D / 32>, dim3(p.hq, p.batch), dim3(kMergeThreads), 0, l.stream, p);
    stage_end(l);
    return e;
}

template <int HKV>
static cudaError_t launch_attend_tc(const LayerParams& p, const Launch& l) {
    constexpr int BPC = HKV == 1 ? 2 : 1;
    const size_t smem = (size_t)2 * BPC * 16 * (HKV * 256 + 16) + (size_t)BPC * 2 * 4096 + 16;
    static SmemConfig configured = {};
    cudaError_t e = ensure_dynamic_smem(attend_split_tc_kernel<HKV, BPC>, smem, configured);
    if (e != cudaSuccess) return e;
    stage_begin(l, kStageAttendSplit);
    e = launch_pdl(attend_split_tc_kernel<HKV, BPC>, dim3((p.attn_chunks + BPC - 1) / BPC, p.batch), dim3(32 * BPC * HKV),
                               smem, l.stream, p);
    stage_end(l);
    if (e != cudaSuccess) return e;
    stage_begin(l, kStageAttendMerge);
    e = launch_pdl(attend_merge_kernel<__nv_bfloat16, 4>, dim3(p.hq, p.batch), dim3(kMergeThreads), 0, l.stream, p);
    stage_end(l);
    return e;
}

cudaError_t launch_attend(const LayerParams& p, const Launch& l) {
    if (p.attn_tc) {
        switch (p.hkv) {
            case 1: return launch_attend_tc<1>(p, l);
            case 2: return launch_attend_tc<2>(p, l);
            case 4: return launch_attend_tc<4>(p, l);
            default: return launch_attend_tc<8>(p, l);
        }
    }
    if (l.dtype == TS_DTYPE_BF16) {
        if (p.d == 128) return launch_attend_t<__nv_bfloat16, 8>(p, l);
        return launch_attend_t<__nv_bfloat16, 4>(p, l);
    }
    if (p.d == 128) return launch_attend_t<float, 8>(p, l);
    return launch_attend_t<float, 4>(p, l);
}

}  // namespace ts
