// Shared declarations of the tokenselect_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tokenselect_b200.h"

namespace ts {

struct SelRecord;

constexpr int kMaxBatch = 256;        // requests per call (plan arrays live in shared memory)
constexpr int kMaxHq = 64;            // query heads per rank
constexpr int kCandAlign = 128;       // each request's candidate region starts on this multiple
constexpr int kHistBins = 2048;       // first radix level: vote bits [30:20]
constexpr int kFusedThreads = 512;    // 1 copy-issuing warp + 8 mma warps + 7 warps that join after scoring
constexpr int kScoreStages = 5;
constexpr int kScoreStageUnits = 128; // (token, kv-head) rows of 256 B per stage
constexpr int kIdxBlock = 1024;       // pool-row indices staged in shared memory at a time
constexpr int kFlagPad = 256;          // per-CTA flags per (parity, source rank) in the tensor-parallel flag pad
constexpr int kMaxTp = 8;
constexpr long long kPushMaxVotes = 600000;  // candidates x peers up to which the votes are pushed (beyond: pulled, half the bytes)
constexpr int kPushMaxTp = 4;             // largest tensor-parallel degree whose votes are pushed (8 bytes per vote and peer) rather than pulled
constexpr int kFusedDynSmem = 196608;    // dynamic shared memory of the selection kernels (5 stages of 34 KB; the tail needs more)
constexpr int kAttnThreads = 256;
constexpr long long kWaitCycles = 2000000000LL;  // bound of every device-side wait (~1 s)

// Everything a kernel of one layer step needs.  Passed by value.
struct LayerParams {
    // configuration
    int hq, hkv, d, group;
    int n_init, n_local, top_k, n_sel;
    int gqa_map, query_cache, kernel_size;
    float theta, sm_scale, logit_cap;
    int n_layers, max_reqs, max_ctx;
    int tp_size;
    // call
    int layer, batch;
    int q_prerot;              // 1: `q` already is the rotated, rounded scoring query (a prefill chunk's fingerprint)
    const void* q;
    const void* k_new;
    const void* v_new;
    const int* out_cache_loc;
    void* k_pool;
    void* v_pool;
    long long pool_rows;
    const int* rtt;
    long long rtt_stride;
    const int* req_pool_indices;
    const int* seq_lens;
    void* out;
    // workspace
    void* q_rot;               // [max_batch, hq*d] dtype: rotated scoring queries
    int* flags;                // [max_batch] TS_FLAG_*
    int* flags_out;            // the caller's copy of the flags (inspection output), or null
    float* cos_terms;          // [max_batch, 4] (q.c, |q|^2, |c|^2, -)
    float* logits;             // [cand_capacity, hq]
    float2* partials;          // [max_batch, part_stride]: per-CTA (max, sum exp) as [grid, hq]
    int part_stride;           // grid*hq rounded up to an even number of float2
    int grid;                  // CTAs of the selection kernel (one per SM)
    int tile_tokens;           // candidates per work tile; fixes which CTA owns which candidates
    float* votes;              // [cand_capacity] head-summed softmax
    float* votes_sel;          // votes exposed for inspection (== votes_final, or the pooled copy)
    float* votes_final;        // votes the selection reads: == votes, or the tensor-parallel sum
    float* votes_pool;         // [cand_capacity] max-pooled votes
    unsigned* hist;            // [max_batch, kHistBins]
    uint2* cand;               // [cand_capacity] (candidate index, vote bits) of the threshold bin
    unsigned* cand_count;      // [max_batch] entries of `cand` per request
    unsigned* sure_count;      // [max_batch, grid] winners above the threshold bin, per CTA
    unsigned* grid_bar;        // [1] self-resetting grid barrier word
    // tensor-parallel exchange over peer memory (mode kModeTpFused)
    float* const* peer_votes;  // [2][kMaxTp] every rank's raw-vote buffer (own included), one set per parity
    unsigned* const* peer_flags;  // [tp_size] every rank's flag pad [2][tp_size][kFlagPad]
    uint2* const* peer_push;   // [2][kMaxTp] every rank's push area [source rank][cand_capacity] of (vote bits, exchange number), one per parity
    int tp_push;               // votes are pushed to the peers with their exchange number attached (tp_size <= kPushMaxTp), else pulled after a flag
    unsigned* cta_epoch;       // [grid] exchanges done so far, kept per CTA: the next one carries count + 1 in
                               // its flags and uses the buffers of parity (count + 1) & 1; all ranks' same-numbered
                               // CTAs count alike, and nothing on the host changes from call to call
    int tp_rank;
    unsigned long long* phase_ts;  // [64] nanosecond timestamps of CTA 0 at the phase boundaries
    int stamps;                // record them (TS_CFG_PHASE_STAMPS); reading %globaltimer is slow, so off by default
    int* sel_slots;            // [max_batch, n_sel]
    int* sel_pos;              // [max_batch, n_sel]
    int* sel_count;            // [max_batch]
    float* attn_o;             // [max_batch, attn_chunks, hq, d]
    float2* attn_ml;           // [max_batch, attn_chunks, hq]
    int attn_chunks;
    int attn_chunk_tokens;
    const float2* score_cs;    // [d/2] (cos, sin) of the scoring position
    const float2* attn_cs;     // [n_sel+1, d/2]
    const float2* attn_cs_lane; // same rows, entries in the order the attention kernel's lanes read them
    const float4* attn_cs_tile; // same rows in 8-position tiles ordered for the tensor-core attention kernel
    int attn_tc;               // 1: tensor-core split kernel (bf16, head_dim 128), chunks of 16 rows
    long long cand_capacity;
    // per-request selection cache
    void* fp_cache;            // [max_reqs, n_layers, hq*d] dtype
    int* pos_cache;            // [max_reqs, n_layers, top_k]
    int* valid;                // [max_reqs, n_layers]
    unsigned long long* counters;  // [max_reqs, 2] retrievals, reuses
    int* err;                  // [2] sticky (code, detail)
    long long wait_cycles;     // bound of every device-side wait, in SM clock cycles
    // attention inside the selection kernel
    int attn_inline;               // 1: phases 5 and 6 run in the selection kernel, no attention kernels follow
    struct SelRecord* records;     // [max_batch, grid] what each CTA found for each request (phase 3)
    float* part_o;                 // [pslots, hq, d] unnormalised partial outputs, one per (request, CTA)
    float2* part_ml;               // [pslots, hq] (max in base-2 units, sum)
    const float* attn_inv_freq;    // [d/2] rotation frequencies of the attention positions (already / rope_scale)
};

static_assert(sizeof(LayerParams) % 4 == 0 && sizeof(LayerParams) / 4 <= kFusedThreads, "one word of the parameters per thread");

// Per-request plan, rebuilt in shared memory by every kernel from seq_lens and flags.
struct Plan {
    int n[kMaxBatch];          // sequence length
    int req[kMaxBatch];        // request slot (row of req_to_token), clamped into range
    int flag[kMaxBatch];
    int nc[kMaxBatch];         // candidates scored this step (0 unless RECOMPUTE)
    int off[kMaxBatch + 1];    // start of the request's candidate region (multiple of kCandAlign)
    int ok;                    // 0: the sticky error word is set, or the workspace is too small
};

__device__ __forceinline__ void set_error(int* err, int code, int detail) {
    if (atomicCAS(err, 0, code) == 0) err[1] = detail;
}

// Number of candidates the selection reads after the optional max-pool: an even window shortens
// the vote vector by one (padding (K-1)/2 on both sides, stride 1).
__host__ __device__ __forceinline__ int pooled_len(int nc, int kernel_size) {
    if (kernel_size <= 0) return nc;
    int pad = (kernel_size - 1) / 2;
    return nc + 2 * pad - kernel_size + 1;
}

// All threads of the block call this; returns after a __syncthreads().  False means: do nothing.
// kGuardOnly: derive the flags from the length guard alone (selection cache off) instead of reading
// the flags a previous phase wrote.
template <bool kGuardOnly = false>
__device__ __forceinline__ bool build_plan(const LayerParams& p, Plan& s) {
#pragma unroll 1
    for (int b = threadIdx.x; b < p.batch; b += blockDim.x) {
        int n = p.seq_lens[b];
        const int req = p.req_pool_indices[b];
        const bool bad = n < 1 || n > p.max_ctx || req < 0 || req >= p.max_reqs;
        int f;
        if (kGuardOnly) {
            f = (bad || p.n_sel >= n) ? TS_FLAG_DENSE : TS_FLAG_RECOMPUTE;
        } else {
            f = __ldcg(p.flags + b);
        }
        s.n[b] = n;
        s.req[b] = bad ? 0 : req;
        s.flag[b] = f;
        s.nc[b] = (f == TS_FLAG_RECOMPUTE) ? (n - p.n_init - p.n_local) : 0;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        int carry = 0;
#pragma unroll 1
        for (int base = 0; base < p.batch; base += 32) {
            int b = base + threadIdx.x;
            int v = (b < p.batch) ? ((s.nc[b] + kCandAlign - 1) / kCandAlign) * kCandAlign : 0;
            int inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, inc, o);
                if ((int)threadIdx.x >= o) inc += t;
            }
            if (b < p.batch) s.off[b] = carry + inc - v;
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (threadIdx.x == 0) {
            s.off[p.batch] = carry;
            s.ok = (*(volatile int*)p.err == 0) ? 1 : 0;
            if ((long long)carry > p.cand_capacity) {
                set_error(p.err, TS_ERR_CAPACITY, carry);
                s.ok = 0;
            }
        }
    }
    __syncthreads();
    return s.ok != 0;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// (max, sum) pairs of an online softmax.
__device__ __forceinline__ void ml_merge(float& m, float& l, float mo, float lo) {
    float mn = fmaxf(m, mo);
    if (mn == -INFINITY) { m = mn; l = 0.f; return; }
    l = l * exp2f((m - mn) * 1.4426950408889634f) + lo * exp2f((mo - mn) * 1.4426950408889634f);
    m = mn;
}

// host-side launchers, one per translation unit ------------------------------------------------
// Optional per-kernel event timing (ts_timing_begin / ts_timing_end).
struct StageTimer {
    cudaEvent_t* events;       // [2 * capacity] start/stop pairs
    int* stages;               // [capacity] stage id of each recorded launch
    int capacity, used, on;
};

struct Launch {
    cudaStream_t stream;
    int num_sms;
    int dtype;
    unsigned flags;
    unsigned long long* launch_count;
    StageTimer* timer;
};

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of a kernel: remember, per
// kernel (one static instance per launcher), the largest size already configured on each device.
struct SmemConfig {
    size_t bytes[64];
};
template <typename F>
inline cudaError_t ensure_dynamic_smem(F func, size_t bytes, SmemConfig& cfg) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (bytes > cfg.bytes[dev]) {
        e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return e;
        cfg.bytes[dev] = bytes;
    }
    return cudaSuccess;
}

enum Stage { kStagePrep = 0, kStageSelect = 1, kStageSelectTpB = 2, kStageAttendSplit = 3, kStageAttendMerge = 4,
             kStageExtendPrep = 5, kStageExtendGather = 6, kStageExtendAttend = 7 };

// Bracket every kernel launch with these two: counts the launch and, when timing is on, records an
// event pair on the launching stream.
inline void stage_begin(const Launch& l, int stage) {
    ++*l.launch_count;
    StageTimer* t = l.timer;
    if (t && t->on && t->used < t->capacity) {
        t->stages[t->used] = stage;
        cudaEventRecord(t->events[2 * t->used], l.stream);
    }
}
inline void stage_end(const Launch& l) {
    StageTimer* t = l.timer;
    if (t && t->on && t->used < t->capacity) {
        cudaEventRecord(t->events[2 * t->used + 1], l.stream);
        ++t->used;
    }
}

cudaError_t launch_rope_tables(float2* score_cs, float2* attn_cs, int d, int n_rows, double base,
                               double rope_scale, int n_local, cudaStream_t stream);
cudaError_t launch_tile_order_table(const float2* attn_cs, float4* attn_cs_tile, int n_rows, int n_tiles, cudaStream_t stream);
cudaError_t launch_lane_order_table(const float2* attn_cs, float2* attn_cs_lane, int d, int n_rows, cudaStream_t stream);

// Position of rotation entry i (0 <= i < d/2) inside a lane-ordered table row: lane j = i / E of an
// eight-lane group owns entries [E*j, E*j+E); its f-th 16-byte load covers entries E*j+2f, E*j+2f+1, and
// the eight lanes' f-th loads are contiguous.  E = d/16.
__host__ __device__ __forceinline__ int lane_order_slot(int i, int e_per_lane) {
    const int j = i / e_per_lane, r = i - j * e_per_lane;
    return ((r >> 1) * 8 + j) * 2 + (r & 1);
}
// Phases the selection kernel runs in one launch.
enum FusedMode {
    kModeAll = 0,   // prepare, score, vote, top-k, emit (single GPU)
    kModeTpA = 1,   // decide, score, vote -> raw votes (before the tensor-parallel sum)
    kModeTpB = 2,   // histogram of the summed votes, top-k, emit
    kModeTpFused = 3,  // like kModeAll, with the vote sum over ranks done in the kernel through peer memory
};

// One prefill chunk of one request (extend.cu).  Shapes and knobs are copied from the handle; the call
// fields come from ts_extend_args; the workspace pointers from the arena.
struct ExtendParams {
    int hq, hkv, d, group;
    int n_init, n_local, n_sel;
    int chunk_len, seq_len, req, layer;
    float sm_scale, logit_cap;
    double rope_base, rope_scale;
    const void* q;              // [chunk_len, hq*d] un-rotated
    const void* k_new;          // [chunk_len, hkv*d] or null
    const void* v_new;
    const int* out_cache_loc;   // [chunk_len]
    void* k_pool;
    void* v_pool;
    long long pool_rows;
    const float2* chunk_cs;     // [chunk_len, d/2] (cos, sin) of positions (n_local + t) * rope_scale, or null
    void* out;                  // [chunk_len, hq*d]
    void* fp;                   // [hq*d] the chunk's scoring query
    int* meta;                  // [2] sequence length, request slot: what the selection kernel reads as its batch
    void* kc;                   // [hkv, rows_k, d] listed keys rotated at their list position
    void* vc;                   // [hkv, rows_k, d] listed values
    void* qc;                   // [hq, rows_q, d] the chunk's queries rotated at their list position
    int rows_k, rows_q;         // padded row counts: multiples of 64 and of 128
    const int* sel_slots;
    const int* sel_count;
    const float2* attn_cs;
    int* err;
    long long wait_cycles;
    unsigned long long* stamps; // TS_CFG_PHASE_STAMPS: where the attention kernel leaves its cycle counts, else null
};

cudaError_t launch_extend_prep(const ExtendParams& e, const Launch& l);
cudaError_t launch_extend_attend(const ExtendParams& e, const Launch& l);
bool extend_uses_tensor_cores(int dtype, int d, int group);
cudaError_t launch_prep(const LayerParams& p, const Launch& l);
cudaError_t launch_fused(const LayerParams& p, const Launch& l, int mode);
cudaError_t launch_attend(const LayerParams& p, const Launch& l);
int fused_grid_size(int num_sms);
bool fused_attends(int dtype, unsigned flags, int hkv, int d, int group, int kernel_size, int grid);
int fused_attn_rows(int hkv);
cudaError_t launch_inv_freq_table(const float2* attn_cs, float* inv_freq, int d, cudaStream_t stream);
int fused_tile_tokens(int dtype, unsigned flags, int hkv, int d, int group);

}  // namespace ts
