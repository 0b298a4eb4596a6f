/*
 * tokenselect_b200 -- C ABI of the decode-time token selection + sparse paged attention path.
 *
 * One library, plain C signatures, device pointers and sizes only.  The host side (Python,
 * ctypes) mirrors the reference's patched attention forward on top of these calls.
 *
 * Conventions
 *   - every call returns an int status (TS_OK == 0); nothing throws;
 *   - calls that take a stream enqueue work on it and return without synchronising the host;
 *   - all tensor pointers are borrowed device pointers that must stay valid until the stream has
 *     passed the call's work; the library owns only its workspace and the per-request selection
 *     cache, both allocated once by ts_create();
 *   - one handle per process and GPU; calls on one handle are not thread-safe (the serving
 *     stack drives a GPU from a single worker thread);
 *   - errors found on the device (a pool row outside the pool, a workspace that is too small, a
 *     bounded wait that ran out) are recorded in a sticky device word: later kernels of the
 *     handle return early until ts_last_error() has read and cleared it.
 *
 * File:line citations name the reference code each entry point replaces
 * (patcher/token_retrieval.py of pzs19/TokenSelect).
 */
#ifndef TOKENSELECT_B200_H
#define TOKENSELECT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TS_ABI_VERSION 3

/* status codes */
#define TS_OK 0
#define TS_ERR_INVALID_ARG 1
#define TS_ERR_UNSUPPORTED 2      /* shape or dtype the kernels are not built for */
#define TS_ERR_CUDA 3             /* a CUDA runtime call failed (see ts_last_cuda_error) */
#define TS_ERR_CAPACITY 4         /* batch / context larger than the workspace was created for */
#define TS_ERR_DEVICE_TIMEOUT 5   /* a bounded device-side wait ran out */
#define TS_ERR_BAD_SLOT 6         /* a pool row index outside [0, pool_rows) */
#define TS_ERR_BAD_LENGTH 7       /* a sequence length outside [1, max_ctx] or a bad request slot */
#define TS_ERR_INTERNAL 8         /* an internal consistency check failed */

/* element type of q, k, v, the pools and the output */
#define TS_DTYPE_BF16 0
#define TS_DTYPE_F32 1            /* check mode: every kernel computes from fp32 inputs */

/* query-head -> KV-head pairing used while scoring (token_retrieval.py:202) */
#define TS_GQA_MOD 0              /* h % hkv: what the reference does */
#define TS_GQA_DIV 1              /* h / (hq/hkv): the conventional map */

/* per-request decision of one layer step, as written to dbg_flags */
#define TS_FLAG_DENSE 0           /* n_init+top_k+n_local >= N: attend to all tokens (:376-378) */
#define TS_FLAG_RECOMPUTE 1       /* scores recomputed                               (:395-417) */
#define TS_FLAG_REUSE 2           /* cached index set reused                         (:418-420) */

/* ts_config.flags */
#define TS_CFG_PLAIN_SCORE 1u     /* score with the plain-load kernel also for bf16 (diagnostic) */
#define TS_CFG_DIRECT_SCORE 2u    /* bf16: load keys straight into mma fragments whatever the row size */
#define TS_CFG_EXTEND_MMA_SYNC 8u /* prefill attention with mma.sync instead of tcgen05 (diagnostic) */
#define TS_CFG_EXTEND_FOUR_PER_ROW 16u /* prefill attention: one softmax team, four threads per query row (diagnostic) */
#define TS_CFG_EXTEND_NARROW_BLOCKS 512u /* prefill attention in 64-key blocks with one issuing thread, two softmax threads per row (the earlier form; diagnostic) */
#define TS_CFG_PHASE_STAMPS 32u   /* kernels record %globaltimer at their phase boundaries for ts_debug_read(3) (diagnostic; off: no timer reads) */
#define TS_CFG_TP_PULL 2048u       /* tensor-parallel exchange: pull the peers' votes after a flag also for tp_size <= 4 (default there: votes pushed with their exchange number attached) */
#define TS_CFG_INLINE_ATTEND 1024u /* attention inside the layer-step kernel also for batches of several requests (default: single requests only) */
#define TS_CFG_SPLIT_ATTEND 256u  /* attention in separate kernels after the selection kernel whatever the shape (diagnostic) */
#define TS_CFG_STAGED_SCORE 4u    /* bf16: stage keys through shared memory by bulk copies whatever the row size */

/*
 * Knobs.  Replaces the module globals written by patch() (token_retrieval.py:885-918), the
 * constructor arguments of ReqToTokenRetriever / TokenRetriever (:117-146, :264-327) and the
 * attention arguments at :815-823.  Head counts are those of this tensor-parallel rank.
 */
typedef struct ts_config {
    uint32_t struct_size;          /* sizeof(ts_config), checked */
    int32_t device;                /* CUDA device ordinal */
    int32_t n_layers;
    int32_t hq;                    /* query heads on this rank            (:461, :580-582) */
    int32_t hkv;                   /* KV heads on this rank               (:462, :583)     */
    int32_t head_dim;
    int32_t dtype;                 /* TS_DTYPE_* */
    int32_t n_init;                /* :912 */
    int32_t n_local;               /* :913 */
    int32_t top_k;                 /* :911 */
    int32_t kernel_size;           /* vote max-pool width, <= 0 off       (:366-369, :914) */
    int32_t query_cache;           /* selection cache on/off              (:918) */
    float similarity_threshold;    /* cosine threshold, fp32              (:313-315) */
    int32_t gqa_map;               /* TS_GQA_* */
    double rope_base;              /* :907 */
    double rope_scale;             /* :908 */
    float sm_scale;                /* attention logit scale               (:818) */
    float logit_cap;               /* soft cap, used when > 0             (:819) */
    int32_t max_reqs;              /* rows of req_to_token == request slots with cache state */
    int32_t max_batch;             /* requests per call */
    int32_t max_ctx;               /* longest sequence                    (:909 max_n_tokens) */
    int64_t max_total_tokens;      /* sum of sequence lengths over one batch */
    int32_t tp_rank;
    int32_t tp_size;
    uint32_t flags;                /* TS_CFG_* */
    int32_t prefill_chunk;         /* longest prefill chunk ts_extend_chunk() accepts (the reference uses
                                    * 512, :917); 0: no prefill workspace is allocated */
    uint32_t wait_limit_us;        /* bound of every device-side wait (grid barriers, copy completions, the
                                    * peers' flags of the tensor-parallel exchange) in microseconds at the
                                    * device's nominal clock; 0: one second.  A wait that runs out sets
                                    * TS_ERR_DEVICE_TIMEOUT and the kernel carries on to its end; while the
                                    * error word is set every later wait of the handle gives up at once */
    uint32_t reserved0;
    /* Optional host tables built the way RotaryEmbedding builds them (:73-96).  NULL: computed
     * by the library from rope_base / rope_scale.
     *   score_cos_sin: [head_dim/2][2] cos,sin at position n_local*rope_scale (:380-388)
     *   attn_cos_sin : [n_init+top_k+n_local+1][head_dim/2][2] for positions 0.. with
     *                  frequencies divided by rope_scale (:820-822) */
    const float* score_cos_sin;
    const float* attn_cos_sin;
} ts_config;

/*
 * One decode step of one layer for a ragged batch.  Replaces the arguments that
 * patched_radix_attention_forward (:827-842) takes from `self`, `q, k, v` and `input_metadata`.
 */
typedef struct ts_decode_args {
    uint32_t struct_size;          /* sizeof(ts_decode_args), checked */
    int32_t layer;
    int32_t batch;
    int32_t reserved;
    const void* q;                 /* [batch, hq*head_dim], un-rotated                      (:816) */
    const void* k_new;             /* [batch, hkv*head_dim] or NULL: rows appended first    (:849) */
    const void* v_new;             /* [batch, hkv*head_dim] or NULL                         (:850) */
    const int32_t* out_cache_loc;  /* [batch] pool rows of the new token                    (:849-852) */
    void* k_pool;                  /* [pool_rows, hkv, head_dim] key buffer of this layer   (:847) */
    void* v_pool;                  /* [pool_rows, hkv, head_dim] value buffer               (:848) */
    int64_t pool_rows;
    const int32_t* req_to_token;   /* [max_reqs, stride]: logical position -> pool row      (:599-601) */
    int64_t req_to_token_stride;   /* elements between rows */
    const int32_t* req_pool_indices; /* [batch] row of req_to_token per request             (:522) */
    const int32_t* seq_lens;       /* [batch] tokens per request, counting the new one      (:523) */
    void* out;                     /* [batch, hq*head_dim]                                  (:825) */
    /* tensor-parallel exchange buffers (tp_size > 1): the caller all-reduces them between the
     * three ts_tp_* calls                                                                  (:363-364) */
    float* tp_votes;               /* >= ts_vote_buffer_elems() floats */
    float* tp_cos;                 /* 4 floats per request: q.c, |q|^2, |c|^2, unused */
    /* optional device outputs for inspection, NULL to skip */
    int32_t* dbg_sel_slots;        /* [batch, n_sel] pool rows attended, list order */
    int32_t* dbg_sel_pos;          /* [batch, n_sel] logical positions */
    int32_t* dbg_sel_count;        /* [batch] */
    int32_t* dbg_flags;            /* [batch] TS_FLAG_* */
    void* stream;                  /* cudaStream_t */
} ts_decode_args;

typedef struct ts_handle ts_handle;

int ts_abi_version(void);
const char* ts_status_string(int status);

/* Device bytes ts_create() will allocate for `cfg` (workspace + selection cache). */
int ts_query_workspace(const ts_config* cfg, size_t* bytes);

/* Elements of the fp32 vote vector for this configuration (size of the tp_votes buffer and of
 * the tensor-parallel all-reduce message). */
int ts_vote_buffer_elems(const ts_config* cfg, int64_t* elems);

/* Allocate workspace and per-request state: replaces ReqToTokenRetriever.__init__ and
 * TokenRetriever.__init__ (:117-146, :264-327). */
int ts_create(const ts_config* cfg, ts_handle** out);
int ts_destroy(ts_handle* h);

/* A request joined or left request slot `req_slot`: forget its cached query, cached index set
 * and counters.  Replaces get_token_retriever()'s fresh TokenRetriever (:147-163, :322-327). */
int ts_reset_request(ts_handle* h, int32_t req_slot, void* stream);

/* Whole layer step in one call: append K/V, select, attend (with tp_size > 1: after ts_tp_attach_peers).  Replaces
 * patched_radix_attention_decode_forward_flashinfer (:777-825) with store_kv_cache (:844-854)
 * and retrieval_indices (:375-449). */
int ts_decode_layer(ts_handle* h, const ts_decode_args* args);

/*
 * One chunk of a prefill of ONE request, one layer.  Replaces one iteration of the chunk loop of
 * patched_radix_attention_extend_forward_flashinfer (:716-775): store the chunk's K/V rows (:726-734),
 * select with the chunk's fingerprint -- the mean over the chunk of the queries rotated at positions
 * n_local, n_local+1, ... and rounded to the model dtype (:380-392, :736-738) -- fall back to all tokens
 * when n_init+top_k+n_local >= seq_len (:741-744), and run causal attention of the chunk's queries over
 * the list, the chunk being the list's tail: query t sees list entries j <= count - chunk_len + t and sits
 * at that position; entry j is rotated at position j (:746-772).  The caller loops over chunks of at most
 * ts_config.prefill_chunk tokens exactly as :716-724 does.
 *
 * Needs prefill_chunk > 0 in the configuration and n_init+top_k+n_local >= chunk_len; with tp_size > 1 the
 * peers must be attached (ts_tp_attach_peers) and the selection cache off, as for ts_decode_layer.
 * The selection cache, when on, is consulted and updated with the fingerprint as in the reference.
 */
typedef struct ts_extend_args {
    uint32_t struct_size;          /* sizeof(ts_extend_args), checked */
    int32_t layer;
    int32_t chunk_len;             /* 1 .. prefill_chunk */
    int32_t req_pool_index;        /* row of req_to_token / request slot (host value) */
    int32_t seq_len;               /* tokens of the request INCLUDING this chunk (host value) */
    int32_t reserved;
    const void* q;                 /* [chunk_len, hq*head_dim], un-rotated */
    const void* k_new;             /* [chunk_len, hkv*head_dim] or NULL (rows already in the pools) */
    const void* v_new;
    const int32_t* out_cache_loc;  /* [chunk_len] pool rows of the chunk's tokens              (:852) */
    void* k_pool;
    void* v_pool;
    int64_t pool_rows;
    const int32_t* req_to_token;
    int64_t req_to_token_stride;
    /* optional device table [chunk_len][head_dim/2][2]: cos, sin of position (n_local + t) * rope_scale
     * built as RotaryEmbedding builds it (:73-96); NULL: computed in the kernel */
    const float* chunk_cos_sin;
    void* out;                     /* [chunk_len, hq*head_dim] */
    /* optional device outputs for inspection, NULL to skip */
    int32_t* dbg_sel_slots;        /* [n_sel] */
    int32_t* dbg_sel_pos;          /* [n_sel] */
    int32_t* dbg_sel_count;        /* [1] */
    int32_t* dbg_flags;            /* [1] */
    void* dbg_fingerprint;         /* [hq*head_dim] model dtype */
    void* stream;
} ts_extend_args;

int ts_extend_chunk(ts_handle* h, const ts_extend_args* args);

/* The same step split at the tensor-parallel exchange points (:363-364):
 *   ts_tp_prepare       K/V append, scoring-query rotation, cosine terms -> args->tp_cos
 *   [caller: all_reduce(tp_cos, SUM) when the selection cache is on]
 *   ts_tp_score_vote    decision, scoring, per-head softmax + head sum  -> args->tp_votes
 *   [caller: all_reduce(tp_votes, SUM)]
 *   ts_tp_select_attend top-k on the reduced votes, union, attention    -> args->out        */
int ts_tp_prepare(ts_handle* h, const ts_decode_args* args);
int ts_tp_score_vote(ts_handle* h, const ts_decode_args* args);
int ts_tp_select_attend(ts_handle* h, const ts_decode_args* args);

/* Tensor-parallel exchange inside the selection kernel (replaces the host-driven all-reduce of
 * :363-364 with loads from the peers' memory over NVLink).  Every rank allocates a buffer of
 * ts_tp_symmetric_bytes() that its peers can address (CUDA IPC / symmetric memory; zero-filled), then
 * passes the device addresses of ALL ranks' buffers, in rank order, to ts_tp_attach_peers().  After that
 * ts_decode_layer() works with tp_size > 1: up to four ranks, each rank stores its raw votes, paired with the
 * exchange's number, straight into its peers' buffers and polls its own buffer for theirs (no flags, no
 * system-scope fence; TS_CFG_TP_PULL selects the other form); above four, each rank writes its raw votes to its
 * own buffer, flags its peers, waits for their flags and loads their votes.  Either way every wait is bounded and
 * the ranks' votes are summed in rank order, so all ranks select from bit-identical sums.  All ranks must issue the same sequence of calls (the exchanges are counted on the
 * device, per CTA, by every launch whether it ran to its end or gave up on a wait, so the ranks' counts stay
 * aligned across a device-side time-out and nothing has to be attached again after one; a rank that creates
 * a NEW handle must pair it with new, zero-filled buffers on every rank).  Not available with the selection
 * cache on (its cosine terms would need a second exchange): use the three ts_tp_* calls then. */
int ts_tp_symmetric_bytes(const ts_config* cfg, size_t* bytes);
int ts_tp_attach_peers(ts_handle* h, const uint64_t* peer_buffers, int32_t count);

/* Selection-cache counters of a request slot (retrieval_count / skip_count, :150-161, :420-421).
 * Synchronises the stream given. */
int ts_get_counters(ts_handle* h, int32_t req_slot, uint64_t* retrievals, uint64_t* reuses, void* stream);

/* Read and clear the sticky device error word.  Synchronises the device.  *code is a TS_ERR_*
 * value or TS_OK; *detail is the offending value (row, length, ...) where one exists. */
int ts_last_error(ts_handle* h, int32_t* code, int32_t* detail);
const char* ts_last_cuda_error(ts_handle* h);

/* Copy an internal buffer of the last call to host memory (synchronises; for tests).
 *   which: 0 rotated scoring queries [batch, hq*head_dim] (dtype)
 *          1 logits  [vote elems, hq] fp32, column c = kv_head*(hq/hkv) + j where j counts the
 *            query heads paired with kv_head in ascending head order
 *          2 votes   [vote elems] fp32 (after max-pool when enabled)
 *          3 sixty-four uint64 nanosecond timestamps left by the kernels at their phase boundaries
 *            (recorded only when ts_config.flags has TS_CFG_PHASE_STAMPS; all zero otherwise)
 *          4 per request [batch] uint32: candidates that shared the vote histogram's threshold bin
 * In 1 and 2 the requests that recomputed their scores follow each other in batch order, each
 * region starting on a multiple of 128 candidates. */
int ts_debug_read(ts_handle* h, int32_t which, void* host_dst, size_t bytes);

/* Number of kernels launched by this handle so far. */
int ts_launch_count(ts_handle* h, uint64_t* launches);

/* Per-kernel device timing with CUDA events recorded on the launching stream around every kernel.
 * ts_timing_begin() allocates the event pool (up to `max_launches` kernels) and switches recording
 * on; ts_timing_end() synchronises, switches it off and returns, per stage, the summed device
 * milliseconds and the number of launches.  Stages: 0 prepare (tensor-parallel form only), 1 the
 * selection kernel (prepare, score, vote, top-k, emit; or its first part under tensor parallelism),
 * 2 its second part under tensor parallelism, 3 attend-split, 4 attend-merge; prefill chunks: 5 append +
 * fingerprint, 6 gather + rotate, 7 causal attention.  The
 * reference's counterpart is the
 * cuda_timer context manager (token_retrieval.py:41-53).  Recording adds an event pair per kernel,
 * so throughput numbers are taken with it off. */
#define TS_NUM_STAGES 8
int ts_timing_begin(ts_handle* h, int32_t max_launches);
int ts_timing_end(ts_handle* h, double* ms_by_stage, uint64_t* launches_by_stage);

/*
 * Sparse paged decode attention over a caller-supplied list of pool rows, for callers that must not
 * allocate.  It has no counterpart in the reference (which allocates freely through torch).
 *
 * Meant for code that runs where device allocation is off limits: a host callback or a serving loop that
 * may not touch the allocator (cudaMalloc can synchronise the device), or a process whose device memory
 * was handed out in full at start-up and whose owner gives out no more.  Such code cannot call ts_create() (one cudaMalloc), so this call takes no handle: the
 * split kernel's partial results live in a fixed 4 MiB array inside the library image (every GPU that
 * loads the library holds it until the process exits).  The call itself performs no cudaMalloc, cudaFree
 * or other allocating call.
 *
 *   - one request per call; `rows` lists `count` pool rows in attention order (the j-th row sits at
 *     position j, the query at position count-1); arithmetic as in ts_decode_layer's attention;
 *   - limit: ceil(count/32) * hq * (head_dim + 2) * 4 bytes <= 4 MiB (e.g. count <= 8064 at hq = 32,
 *     head_dim = 128); longer lists return TS_ERR_CAPACITY;
 *   - the array is shared by all calls and keeps the last call's contents; nothing in it needs clearing
 *     (each call writes every partial it later reads), but two calls whose kernels overlap on the GPU
 *     race on it -- order them on one stream or with events;
 *   - the first call on a device looks up the array's device address; make that first call before any
 *     stream capture begins, and from one thread: the per-device address table behind this call is not
 *     guarded, so two threads making the first call on a device at the same time race on it (later calls
 *     only read it);
 *   - `status`, if not NULL, is a device int the kernels set to TS_ERR_BAD_SLOT when a listed row lies
 *     outside [0, pool_rows) (that row is then read as row 0).
 */
typedef struct ts_attend_static_args {
    uint32_t struct_size;          /* sizeof(ts_attend_static_args), checked */
    int32_t dtype;                 /* TS_DTYPE_* of q, the pools and out */
    int32_t hq;                    /* query heads */
    int32_t hkv;                   /* KV heads; hq / hkv <= 8 */
    int32_t head_dim;              /* 64 or 128 */
    int32_t count;                 /* listed rows */
    const void* q;                 /* [hq*head_dim], un-rotated */
    const void* k_pool;            /* [pool_rows, hkv, head_dim] */
    const void* v_pool;            /* [pool_rows, hkv, head_dim] */
    int64_t pool_rows;
    const int32_t* rows;           /* [count] pool rows, device memory */
    void* out;                     /* [hq*head_dim] */
    float sm_scale;
    float logit_cap;               /* soft cap, used when > 0 */
    double rope_base;
    double rope_scale;
    int32_t* status;               /* optional device int, see above */
    void* stream;                  /* cudaStream_t */
} ts_attend_static_args;

int ts_attend_rows_static(const ts_attend_static_args* args);

#ifdef __cplusplus
}
#endif
#endif /* TOKENSELECT_B200_H */
