// C ABI of tokenselect_b200: handle, workspace, call sequencing.  See include/tokenselect_b200.h.
#include <stdio.h>
#include <string.h>

#include <new>

#include "common.cuh"

using namespace ts;

struct ts_handle {
    ts_config cfg;
    int num_sms;
    int n_sel;
    size_t elem;                  // bytes per element of the model dtype
    long long cand_capacity;
    int grid;
    int attn_chunk_tokens, attn_chunks;
    // one device allocation, carved up
    unsigned char* arena;
    size_t arena_bytes;
    LayerParams base;             // workspace pointers and configuration, call fields empty
    unsigned long long launches;
    StageTimer timer;
    // tensor-parallel exchange through peer memory
    bool peers_attached;
    unsigned* dev_cta_epoch;                // [grid] exchanges done, per CTA
    unsigned char* peer_base[kMaxTp];      // every rank's symmetric buffer (host copy)
    float** dev_peer_votes;                 // [2][kMaxTp] device array of pointers
    uint2** dev_peer_push;                  // [2][kMaxTp]
    unsigned** dev_peer_flags;              // [kMaxTp]
    int last_batch;
    long long wait_cycles;                  // ts_config.wait_limit_us in SM clock cycles
    // prefill chunks
    void* ext_fp; int* ext_meta; void* ext_k; void* ext_v; void* ext_q;
    int ext_rows_k, ext_rows_q;
    char cuda_msg[256];
};

namespace {

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int validate(const ts_config* c) {
    if (!c || c->struct_size != sizeof(ts_config)) return TS_ERR_INVALID_ARG;
    if (c->n_layers < 1 || c->hq < 1 || c->hkv < 1 || c->hq % c->hkv != 0) return TS_ERR_INVALID_ARG;
    if (c->hq > kMaxHq) return TS_ERR_UNSUPPORTED;
    if (c->head_dim != 64 && c->head_dim != 128) return TS_ERR_UNSUPPORTED;
    if (c->dtype != TS_DTYPE_BF16 && c->dtype != TS_DTYPE_F32) return TS_ERR_UNSUPPORTED;
    if (c->hq / c->hkv > 8) return TS_ERR_UNSUPPORTED;
    if (c->n_init < 0 || c->n_local < 1 || c->top_k < 1) return TS_ERR_INVALID_ARG;
    if (c->max_reqs < 1 || c->max_batch < 1 || c->max_batch > kMaxBatch) return TS_ERR_INVALID_ARG;
    if (c->max_ctx < 1 || c->max_total_tokens < 1) return TS_ERR_INVALID_ARG;
    if (c->gqa_map != TS_GQA_MOD && c->gqa_map != TS_GQA_DIV) return TS_ERR_INVALID_ARG;
    if (c->tp_size < 1 || c->tp_rank < 0 || c->tp_rank >= c->tp_size) return TS_ERR_INVALID_ARG;
    if (c->tp_size > kMaxTp) return TS_ERR_UNSUPPORTED;       // the peer tables hold kMaxTp ranks
    if (!(c->rope_base > 0.0) || !(c->rope_scale > 0.0)) return TS_ERR_INVALID_ARG;
    if (c->prefill_chunk < 0 || c->prefill_chunk > 4096) return TS_ERR_INVALID_ARG;
    return TS_OK;
}

long long cand_capacity_of(const ts_config* c) {
    // every request's candidate region is rounded up to kCandAlign
    return (long long)align_up((size_t)c->max_total_tokens, kCandAlign) + (long long)kCandAlign * c->max_batch;
}

struct Carve {
    size_t off = 0;
    size_t take(size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; }
};

// Computes the arena layout; with h == nullptr only the total is produced.
size_t layout(const ts_config* c, int num_sms, ts_handle* h) {
    const size_t elem = c->dtype == TS_DTYPE_BF16 ? 2 : 4;
    const int n_sel = c->n_init + c->top_k + c->n_local;
    const long long cap = cand_capacity_of(c);
    const int grid = fused_grid_size(num_sms);
    const size_t hd = (size_t)c->hq * c->head_dim;
    // split the list so that one request's chunks fill the SMs once (tokens go in groups of four;
    // the staged K/V rows of a chunk must fit in shared memory)
    int ch = (n_sel + num_sms - 1) / num_sms;
    ch = ch < 16 ? 16 : (ch + 3) / 4 * 4;
    while (ch > 4 && (size_t)ch * 2 * c->hkv * c->head_dim * elem > 160 * 1024) ch -= 4;
    // bf16 at head_dim 128 runs the tensor-core split kernel: partials per 16 listed rows
    const bool attn_tc = c->dtype == TS_DTYPE_BF16 && c->head_dim == 128 && c->hq / c->hkv <= 8 &&
                         (c->hkv == 1 || c->hkv == 2 || c->hkv == 4 || c->hkv == 8);
    if (attn_tc) ch = 16;
    const int cs_tiles = (n_sel + 1 + 15) / 16 * 2;
    const int chunks = (n_sel + ch - 1) / ch;
    Carve cv;
    size_t o_err = cv.take(16);
    size_t o_qrot = cv.take((size_t)c->max_batch * hd * elem);
    size_t o_flags = cv.take((size_t)c->max_batch * 4);
    size_t o_cos = cv.take((size_t)c->max_batch * 16);
    size_t o_logits = cv.take((size_t)cap * c->hq * 4);
    const int part_stride = (grid * c->hq + 1) & ~1;
    size_t o_part = cv.take((size_t)c->max_batch * part_stride * 8);
    size_t o_votes = cv.take((size_t)cap * 4);
    size_t o_vpool = cv.take(c->kernel_size > 0 ? (size_t)cap * 4 : 16);
    size_t o_hist = cv.take((size_t)c->max_batch * kHistBins * 4);
    size_t o_ccount = cv.take((size_t)c->max_batch * 4);
    size_t o_sure = cv.take((size_t)c->max_batch * grid * 4);
    size_t o_bar = cv.take(16);
    size_t o_ts = cv.take(128 * 8);
    size_t o_pv = cv.take(2 * kMaxTp * sizeof(void*));
    size_t o_pf = cv.take(kMaxTp * sizeof(void*));
    size_t o_pp = cv.take(2 * kMaxTp * sizeof(void*));
    size_t o_ep = cv.take((size_t)grid * 4);
    size_t o_cand = cv.take((size_t)cap * 8);
    size_t o_slots = cv.take((size_t)c->max_batch * n_sel * 4);
    size_t o_pos = cv.take((size_t)c->max_batch * n_sel * 4);
    size_t o_count = cv.take((size_t)c->max_batch * 4);
    size_t o_ao = cv.take((size_t)c->max_batch * chunks * hd * 4);
    size_t o_aml = cv.take((size_t)c->max_batch * chunks * c->hq * 8);
    size_t o_scs = cv.take((size_t)(c->head_dim / 2) * 8);
    size_t o_acs = cv.take((size_t)(n_sel + 1) * (c->head_dim / 2) * 8);
    size_t o_acsl = cv.take((size_t)(n_sel + 1) * (c->head_dim / 2) * 8);
    size_t o_acst = cv.take(attn_tc ? (size_t)cs_tiles * 4096 : 16);
    size_t o_fp = cv.take((size_t)c->max_reqs * c->n_layers * hd * elem);
    size_t o_pc = cv.take((size_t)c->max_reqs * c->n_layers * c->top_k * 4);
    size_t o_valid = cv.take((size_t)c->max_reqs * c->n_layers * 4);
    size_t o_cnt = cv.take((size_t)c->max_reqs * 16);
    // prefill chunks: fingerprint, (length, slot) pair, compact rotated K / V / Q arrays
    const int ext = c->prefill_chunk;
    const int rows_k = (n_sel + 127) / 128 * 128, rows_q = (ext + 127) / 128 * 128;
    size_t o_xfp = cv.take(ext > 0 ? hd * elem : 16);
    size_t o_xmeta = cv.take(16);
    size_t o_xk = cv.take(ext > 0 ? (size_t)c->hkv * rows_k * c->head_dim * elem : 16);
    size_t o_xv = cv.take(ext > 0 ? (size_t)c->hkv * rows_k * c->head_dim * elem : 16);
    size_t o_xq = cv.take(ext > 0 ? (size_t)c->hq * rows_q * c->head_dim * elem : 16);
    // attention inside the selection kernel: per-(request, CTA) records, partials, rotation frequencies
    const bool inl = fused_attends(c->dtype, c->flags, c->hkv, c->head_dim, c->hq / c->hkv, c->kernel_size, grid);
    const int arows = fused_attn_rows(c->hkv);
    const size_t pslots = inl ? (size_t)grid + (size_t)c->max_batch * (2 + (n_sel + arows - 1) / arows) : 1;
    size_t o_rec = cv.take((size_t)c->max_batch * grid * 128);
    size_t o_po = cv.take(pslots * hd * 4);
    size_t o_pml = cv.take(pslots * c->hq * 8);
    size_t o_inv = cv.take((size_t)(c->head_dim / 2) * 4);
    if (h) {
        unsigned char* a = h->arena;
        LayerParams& p = h->base;
        memset(&p, 0, sizeof(p));
        p.hq = c->hq; p.hkv = c->hkv; p.d = c->head_dim; p.group = c->hq / c->hkv;
        p.n_init = c->n_init; p.n_local = c->n_local; p.top_k = c->top_k; p.n_sel = n_sel;
        p.gqa_map = c->gqa_map; p.query_cache = c->query_cache ? 1 : 0; p.kernel_size = c->kernel_size;
        p.theta = c->similarity_threshold; p.sm_scale = c->sm_scale; p.logit_cap = c->logit_cap;
        p.n_layers = c->n_layers; p.max_reqs = c->max_reqs; p.max_ctx = c->max_ctx; p.tp_size = c->tp_size;
        p.err = reinterpret_cast<int*>(a + o_err);
        p.q_rot = a + o_qrot;
        p.flags = reinterpret_cast<int*>(a + o_flags);
        p.cos_terms = reinterpret_cast<float*>(a + o_cos);
        p.logits = reinterpret_cast<float*>(a + o_logits);
        p.partials = reinterpret_cast<float2*>(a + o_part);
        p.grid = grid;
        p.part_stride = part_stride;
        p.tile_tokens = fused_tile_tokens(c->dtype, c->flags, c->hkv, c->head_dim, c->hq / c->hkv);
        p.votes = reinterpret_cast<float*>(a + o_votes);
        p.votes_pool = reinterpret_cast<float*>(a + o_vpool);
        p.votes_sel = c->kernel_size > 0 ? p.votes_pool : p.votes;
        p.votes_final = p.votes;
        p.tp_rank = c->tp_rank;
        p.hist = reinterpret_cast<unsigned*>(a + o_hist);
        p.cand_count = reinterpret_cast<unsigned*>(a + o_ccount);
        p.sure_count = reinterpret_cast<unsigned*>(a + o_sure);
        p.grid_bar = reinterpret_cast<unsigned*>(a + o_bar);
        p.phase_ts = reinterpret_cast<unsigned long long*>(a + o_ts);
        p.stamps = (c->flags & TS_CFG_PHASE_STAMPS) ? 1 : 0;
        h->dev_peer_votes = reinterpret_cast<float**>(a + o_pv);
        h->dev_peer_flags = reinterpret_cast<unsigned**>(a + o_pf);
        h->dev_peer_push = reinterpret_cast<uint2**>(a + o_pp);
        h->dev_cta_epoch = reinterpret_cast<unsigned*>(a + o_ep);
        p.cand = reinterpret_cast<uint2*>(a + o_cand);
        p.sel_slots = reinterpret_cast<int*>(a + o_slots);
        p.sel_pos = reinterpret_cast<int*>(a + o_pos);
        p.sel_count = reinterpret_cast<int*>(a + o_count);
        p.attn_o = reinterpret_cast<float*>(a + o_ao);
        p.attn_ml = reinterpret_cast<float2*>(a + o_aml);
        p.attn_chunks = chunks; p.attn_chunk_tokens = ch;
        p.score_cs = reinterpret_cast<const float2*>(a + o_scs);
        p.attn_cs = reinterpret_cast<const float2*>(a + o_acs);
        p.attn_cs_lane = reinterpret_cast<const float2*>(a + o_acsl);
        p.attn_cs_tile = reinterpret_cast<const float4*>(a + o_acst);
        p.attn_tc = attn_tc ? 1 : 0;
        p.cand_capacity = cap;
        p.fp_cache = a + o_fp;
        p.pos_cache = reinterpret_cast<int*>(a + o_pc);
        p.valid = reinterpret_cast<int*>(a + o_valid);
        p.counters = reinterpret_cast<unsigned long long*>(a + o_cnt);
        p.attn_inline = inl ? 1 : 0;
        p.records = reinterpret_cast<SelRecord*>(a + o_rec);
        p.part_o = reinterpret_cast<float*>(a + o_po);
        p.part_ml = reinterpret_cast<float2*>(a + o_pml);
        p.attn_inv_freq = reinterpret_cast<const float*>(a + o_inv);
        h->ext_fp = a + o_xfp; h->ext_meta = reinterpret_cast<int*>(a + o_xmeta);
        h->ext_k = a + o_xk; h->ext_v = a + o_xv; h->ext_q = a + o_xq;
        h->ext_rows_k = rows_k; h->ext_rows_q = rows_q;
        h->elem = elem; h->n_sel = n_sel; h->cand_capacity = cap; h->grid = grid;
        h->attn_chunk_tokens = ch; h->attn_chunks = chunks;
    }
    return cv.off;
}

bool n_sel_rows_ok(const ts_handle* h) { return h->n_sel >= 1; }   // the table has a row for position 1

int cuda_fail(ts_handle* h, cudaError_t e, const char* what) {
    if (h) snprintf(h->cuda_msg, sizeof(h->cuda_msg), "%s: %s", what, cudaGetErrorString(e));
    return TS_ERR_CUDA;
}

int num_sms_of(int device, int* out) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return TS_ERR_CUDA;
    *out = prop.multiProcessorCount;
    return TS_OK;
}

size_t sym_flag_bytes() { return (size_t)2 * kMaxTp * kFlagPad * sizeof(unsigned); }
size_t sym_votes_offset(long long cap, int parity) { return sym_flag_bytes() + (size_t)parity * (size_t)cap * sizeof(float); }
// Push area (tensor-parallel degrees up to kPushMaxTp): per parity, one slice of cand_capacity (vote, number) pairs
// per source rank.
bool tp_pushes(const ts_config* c) { return c->tp_size > 1 && c->tp_size <= kPushMaxTp && !(c->flags & TS_CFG_TP_PULL); }
size_t sym_push_offset(long long cap, int tp, int parity) {
    return ((sym_votes_offset(cap, 2) + 255) & ~(size_t)255) + (size_t)parity * (size_t)tp * (size_t)cap * sizeof(uint2);
}
size_t sym_total_bytes(const ts_config* c, long long cap) {
    return tp_pushes(c) ? sym_push_offset(cap, c->tp_size, 2) : sym_votes_offset(cap, 2);
}

int fill(ts_handle* h, const ts_decode_args* a, LayerParams& p, Launch& l, bool fused_tp = false) {
    if (!h || !a || a->struct_size != sizeof(ts_decode_args)) return TS_ERR_INVALID_ARG;
    if (a->layer < 0 || a->layer >= h->cfg.n_layers) return TS_ERR_INVALID_ARG;
    if (a->batch < 1) return TS_ERR_INVALID_ARG;
    if (a->batch > h->cfg.max_batch) return TS_ERR_CAPACITY;
    if (!a->q || !a->k_pool || !a->v_pool || !a->req_to_token || !a->req_pool_indices || !a->seq_lens || !a->out)
        return TS_ERR_INVALID_ARG;
    if ((a->k_new != nullptr) != (a->v_new != nullptr)) return TS_ERR_INVALID_ARG;
    if (a->k_new && !a->out_cache_loc) return TS_ERR_INVALID_ARG;
    if (a->pool_rows < 1 || a->req_to_token_stride < 1) return TS_ERR_INVALID_ARG;
    p = h->base;
    p.layer = a->layer; p.batch = a->batch;
    p.q = a->q; p.k_new = a->k_new; p.v_new = a->v_new; p.out_cache_loc = a->out_cache_loc;
    p.k_pool = a->k_pool; p.v_pool = a->v_pool; p.pool_rows = a->pool_rows;
    p.rtt = a->req_to_token; p.rtt_stride = a->req_to_token_stride;
    p.req_pool_indices = a->req_pool_indices; p.seq_lens = a->seq_lens; p.out = a->out;
    p.flags_out = a->dbg_flags;
    if (h->cfg.tp_size > 1 && !fused_tp) {
        if (!a->tp_votes || !a->tp_cos) return TS_ERR_INVALID_ARG;
        p.votes = a->tp_votes;
        p.votes_final = a->tp_votes;
        p.cos_terms = a->tp_cos;
        if (h->cfg.kernel_size <= 0) p.votes_sel = p.votes;
    }
    if (fused_tp) {
        // raw votes go to this rank's peer-visible buffer (the kernel alternates between two per exchange, so
        // that a fast rank never overwrites votes a slow peer is still reading); the sum lands in the workspace
        p.peer_votes = h->dev_peer_votes;
        p.peer_flags = h->dev_peer_flags;
        p.peer_push = h->dev_peer_push;
        p.tp_push = tp_pushes(&h->cfg) ? 1 : 0;
        p.cta_epoch = h->dev_cta_epoch;
        p.votes_final = h->base.votes;
    }
    l.stream = reinterpret_cast<cudaStream_t>(a->stream);
    l.num_sms = h->num_sms;
    l.dtype = h->cfg.dtype;
    l.flags = h->cfg.flags;
    l.launch_count = &h->launches;
    l.timer = &h->timer;
    h->last_batch = a->batch;
    return TS_OK;
}

int copy_debug(ts_handle* h, const ts_decode_args* a, const LayerParams& p, cudaStream_t s) {
    cudaError_t e = cudaSuccess;
    const size_t nb = (size_t)a->batch;
    if (a->dbg_sel_slots && e == cudaSuccess)
        e = cudaMemcpyAsync(a->dbg_sel_slots, p.sel_slots, nb * h->n_sel * 4, cudaMemcpyDeviceToDevice, s);
    if (a->dbg_sel_pos && e == cudaSuccess)
        e = cudaMemcpyAsync(a->dbg_sel_pos, p.sel_pos, nb * h->n_sel * 4, cudaMemcpyDeviceToDevice, s);
    if (a->dbg_sel_count && e == cudaSuccess)
        e = cudaMemcpyAsync(a->dbg_sel_count, p.sel_count, nb * 4, cudaMemcpyDeviceToDevice, s);
    // (dbg_flags: written by the kernels themselves through LayerParams::flags_out)
    return e == cudaSuccess ? TS_OK : cuda_fail(h, e, "debug copy");
}

#define TS_TRY(expr, what)                                     \
    do {                                                       \
        cudaError_t e__ = (expr);                              \
        if (e__ != cudaSuccess) return cuda_fail(h, e__, what); \
    } while (0)

}  // namespace

extern "C" {

int ts_abi_version(void) { return TS_ABI_VERSION; }

const char* ts_status_string(int s) {
    switch (s) {
        case TS_OK: return "ok";
        case TS_ERR_INVALID_ARG: return "invalid argument";
        case TS_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case TS_ERR_CUDA: return "CUDA runtime error";
        case TS_ERR_CAPACITY: return "batch or context exceeds the workspace";
        case TS_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case TS_ERR_BAD_SLOT: return "pool row index outside the pool";
        case TS_ERR_BAD_LENGTH: return "sequence length or request slot out of range";
        case TS_ERR_INTERNAL: return "internal consistency check failed";
    }
    return "unknown status";
}

int ts_query_workspace(const ts_config* cfg, size_t* bytes) {
    int s = validate(cfg);
    if (s != TS_OK) return s;
    if (!bytes) return TS_ERR_INVALID_ARG;
    int sms = 148;
    int dev_count = 0;
    if (cudaGetDeviceCount(&dev_count) == cudaSuccess && cfg->device < dev_count) num_sms_of(cfg->device, &sms);
    *bytes = layout(cfg, sms, nullptr);
    return TS_OK;
}

int ts_vote_buffer_elems(const ts_config* cfg, int64_t* elems) {
    int s = validate(cfg);
    if (s != TS_OK) return s;
    if (!elems) return TS_ERR_INVALID_ARG;
    *elems = cand_capacity_of(cfg);
    return TS_OK;
}

int ts_create(const ts_config* cfg, ts_handle** out) {
    int s = validate(cfg);
    if (s != TS_OK) return s;
    if (!out) return TS_ERR_INVALID_ARG;
    *out = nullptr;
    if (cudaSetDevice(cfg->device) != cudaSuccess) return TS_ERR_CUDA;
    ts_handle* h = new (std::nothrow) ts_handle();
    if (!h) return TS_ERR_CUDA;
    memset(h, 0, sizeof(*h));
    h->cfg = *cfg;
    h->cfg.score_cos_sin = nullptr;
    h->cfg.attn_cos_sin = nullptr;
    if (num_sms_of(cfg->device, &h->num_sms) != TS_OK) { delete h; return TS_ERR_CUDA; }
    // one flag per CTA and source rank in the tensor-parallel flag pad; one record per CTA in the top-k's scratch
    if (fused_grid_size(h->num_sms) > kFlagPad) { delete h; return TS_ERR_UNSUPPORTED; }
    int clock_khz = 0;
    if (cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, cfg->device) != cudaSuccess || clock_khz <= 0)
        clock_khz = 2000000;
    h->wait_cycles = cfg->wait_limit_us ? (long long)cfg->wait_limit_us * clock_khz / 1000 : kWaitCycles;
    h->arena_bytes = layout(cfg, h->num_sms, nullptr);
    if (cudaMalloc(&h->arena, h->arena_bytes) != cudaSuccess) { delete h; return TS_ERR_CUDA; }
    layout(cfg, h->num_sms, h);
    h->base.wait_cycles = h->wait_cycles;
    const LayerParams& p = h->base;
    const int half = cfg->head_dim / 2;
    cudaError_t e = cudaMemset(h->arena, 0, h->arena_bytes);
    // rotation tables: taken from the caller when given, otherwise computed on the device
    if (e == cudaSuccess && (!cfg->score_cos_sin || !cfg->attn_cos_sin))
        e = launch_rope_tables(const_cast<float2*>(p.score_cs), const_cast<float2*>(p.attn_cs), cfg->head_dim,
                               h->n_sel + 1, cfg->rope_base, cfg->rope_scale, cfg->n_local, 0);
    if (e == cudaSuccess && cfg->score_cos_sin)
        e = cudaMemcpy(const_cast<float2*>(p.score_cs), cfg->score_cos_sin, (size_t)half * 8, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && cfg->attn_cos_sin)
        e = cudaMemcpy(const_cast<float2*>(p.attn_cs), cfg->attn_cos_sin, (size_t)(h->n_sel + 1) * half * 8,
                       cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
        e = launch_lane_order_table(p.attn_cs, const_cast<float2*>(p.attn_cs_lane), cfg->head_dim, h->n_sel + 1, 0);
    if (e == cudaSuccess && p.attn_tc)
        e = launch_tile_order_table(p.attn_cs, const_cast<float4*>(p.attn_cs_tile), h->n_sel + 1,
                                    (h->n_sel + 1 + 15) / 16 * 2, 0);
    if (e == cudaSuccess && n_sel_rows_ok(h))
        e = launch_inv_freq_table(p.attn_cs, const_cast<float*>(p.attn_inv_freq), cfg->head_dim, 0);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { cudaFree(h->arena); delete h; return TS_ERR_CUDA; }
    *out = h;
    return TS_OK;
}

static void free_timer(ts_handle* h) {
    for (int i = 0; i < 2 * h->timer.capacity; ++i) cudaEventDestroy(h->timer.events[i]);
    delete[] h->timer.events;
    delete[] h->timer.stages;
    memset(&h->timer, 0, sizeof(h->timer));
}

int ts_destroy(ts_handle* h) {
    if (!h) return TS_ERR_INVALID_ARG;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    free_timer(h);
    cudaFree(h->arena);
    delete h;
    return TS_OK;
}

int ts_reset_request(ts_handle* h, int32_t req_slot, void* stream) {
    if (!h || req_slot < 0 || req_slot >= h->cfg.max_reqs) return TS_ERR_INVALID_ARG;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    TS_TRY(cudaMemsetAsync(h->base.valid + (size_t)req_slot * h->cfg.n_layers, 0, (size_t)h->cfg.n_layers * 4, s),
           "reset valid");
    TS_TRY(cudaMemsetAsync(h->base.counters + 2 * (size_t)req_slot, 0, 16, s), "reset counters");
    return TS_OK;
}

int ts_tp_prepare(ts_handle* h, const ts_decode_args* a) {
    LayerParams p; Launch l;
    int s = fill(h, a, p, l);
    if (s != TS_OK) return s;
    TS_TRY(launch_prep(p, l), "prepare");
    return TS_OK;
}

int ts_tp_score_vote(ts_handle* h, const ts_decode_args* a) {
    LayerParams p; Launch l;
    int s = fill(h, a, p, l);
    if (s != TS_OK) return s;
    p.attn_inline = 0;
    TS_TRY(launch_fused(p, l, kModeTpA), "score+vote");
    return TS_OK;
}

int ts_tp_select_attend(ts_handle* h, const ts_decode_args* a) {
    LayerParams p; Launch l;
    int s = fill(h, a, p, l);
    if (s != TS_OK) return s;
    p.attn_inline = 0;
    TS_TRY(launch_fused(p, l, kModeTpB), "select");
    TS_TRY(launch_attend(p, l), "attend");
    return copy_debug(h, a, p, l.stream);
}

int ts_tp_symmetric_bytes(const ts_config* cfg, size_t* bytes) {
    int s = validate(cfg);
    if (s != TS_OK) return s;
    if (!bytes) return TS_ERR_INVALID_ARG;
    *bytes = sym_total_bytes(cfg, cand_capacity_of(cfg));
    return TS_OK;
}

int ts_tp_attach_peers(ts_handle* h, const uint64_t* peer_buffers, int32_t count) {
    if (!h || !peer_buffers || count != h->cfg.tp_size || count > kMaxTp) return TS_ERR_INVALID_ARG;
    float* votes[2 * kMaxTp] = {nullptr};
    unsigned* flags[kMaxTp] = {nullptr};
    uint2* push[2 * kMaxTp] = {nullptr};
    for (int r = 0; r < count; ++r) {
        if (!peer_buffers[r]) return TS_ERR_INVALID_ARG;
        h->peer_base[r] = reinterpret_cast<unsigned char*>(peer_buffers[r]);
        flags[r] = reinterpret_cast<unsigned*>(h->peer_base[r]);
        for (int par = 0; par < 2; ++par) {
            votes[par * kMaxTp + r] = reinterpret_cast<float*>(h->peer_base[r] + sym_votes_offset(h->cand_capacity, par));
            if (tp_pushes(&h->cfg))
                push[par * kMaxTp + r] = reinterpret_cast<uint2*>(h->peer_base[r] + sym_push_offset(h->cand_capacity, count, par));
        }
    }
    TS_TRY(cudaMemcpy(h->dev_peer_votes, votes, sizeof(votes), cudaMemcpyHostToDevice), "peer table");
    TS_TRY(cudaMemcpy(h->dev_peer_flags, flags, sizeof(flags), cudaMemcpyHostToDevice), "peer table");
    TS_TRY(cudaMemcpy(h->dev_peer_push, push, sizeof(push), cudaMemcpyHostToDevice), "peer table");
    // The per-CTA exchange counts are NOT restarted: every launch of every rank counts, also one that gave
    // up on a wait, so the ranks stay aligned and a flag left in a pad by an earlier exchange can never equal
    // a later exchange's number.
    h->peers_attached = true;
    return TS_OK;
}

int ts_decode_layer(ts_handle* h, const ts_decode_args* a) {
    const bool fused_tp = h && h->cfg.tp_size > 1;
    if (fused_tp) {
        // needs the peers' buffers; the cosine terms of the selection cache are not exchanged in this form
        if (!h->peers_attached) return TS_ERR_INVALID_ARG;
        if (h->cfg.query_cache) return TS_ERR_UNSUPPORTED;
    }
    LayerParams p; Launch l;
    int s = fill(h, a, p, l, fused_tp);
    if (s != TS_OK) return s;
    // The layer-step kernel attends inside the CTAs that own the winners, which pays when a request's candidates
    // span the whole grid.  In a batch every request spans a fraction of the grid only (a short one a CTA or two,
    // which would then attend to all its winners alone), so batches take the selection kernel and the attention
    // kernels, whose grid covers every (request, row block) -- unless TS_CFG_INLINE_ATTEND asks otherwise.
    if (a->batch > 1 && !(h->cfg.flags & TS_CFG_INLINE_ATTEND)) p.attn_inline = 0;
    TS_TRY(launch_fused(p, l, fused_tp ? kModeTpFused : kModeAll), "select");
    if (!p.attn_inline) TS_TRY(launch_attend(p, l), "attend");
    return copy_debug(h, a, p, l.stream);
}

int ts_extend_chunk(ts_handle* h, const ts_extend_args* a) {
    if (!h || !a || a->struct_size != sizeof(ts_extend_args)) return TS_ERR_INVALID_ARG;
    const ts_config& c = h->cfg;
    if (c.prefill_chunk < 1) return TS_ERR_UNSUPPORTED;
    // tensor parallel: only the form that sums the votes inside the selection kernel
    const bool fused_tp = c.tp_size > 1;
    if (fused_tp && (!h->peers_attached || c.query_cache)) return TS_ERR_UNSUPPORTED;
    if (a->layer < 0 || a->layer >= c.n_layers) return TS_ERR_INVALID_ARG;
    if (a->chunk_len < 1) return TS_ERR_INVALID_ARG;
    if (a->chunk_len > c.prefill_chunk) return TS_ERR_CAPACITY;
    if (a->req_pool_index < 0 || a->req_pool_index >= c.max_reqs) return TS_ERR_INVALID_ARG;
    if (a->seq_len < a->chunk_len) return TS_ERR_INVALID_ARG;
    if (a->seq_len > c.max_ctx || a->seq_len > c.max_total_tokens) return TS_ERR_CAPACITY;
    if (!a->q || !a->k_pool || !a->v_pool || !a->req_to_token || !a->out) return TS_ERR_INVALID_ARG;
    if ((a->k_new != nullptr) != (a->v_new != nullptr)) return TS_ERR_INVALID_ARG;
    if (a->k_new && !a->out_cache_loc) return TS_ERR_INVALID_ARG;
    if (a->pool_rows < 1 || a->req_to_token_stride < 1) return TS_ERR_INVALID_ARG;
    // the chunk must fit inside the list it closes (otherwise its first queries would see no key at all)
    if (h->n_sel < a->chunk_len) return TS_ERR_UNSUPPORTED;

    ExtendParams e;
    memset(&e, 0, sizeof(e));
    e.hq = c.hq; e.hkv = c.hkv; e.d = c.head_dim; e.group = c.hq / c.hkv;
    e.n_init = c.n_init; e.n_local = c.n_local; e.n_sel = h->n_sel;
    e.chunk_len = a->chunk_len; e.seq_len = a->seq_len; e.req = a->req_pool_index; e.layer = a->layer;
    e.sm_scale = c.sm_scale; e.logit_cap = c.logit_cap; e.rope_base = c.rope_base; e.rope_scale = c.rope_scale;
    e.q = a->q; e.k_new = a->k_new; e.v_new = a->v_new; e.out_cache_loc = a->out_cache_loc;
    e.k_pool = a->k_pool; e.v_pool = a->v_pool; e.pool_rows = a->pool_rows;
    e.chunk_cs = reinterpret_cast<const float2*>(a->chunk_cos_sin);
    e.out = a->out;
    e.fp = h->ext_fp; e.meta = h->ext_meta; e.kc = h->ext_k; e.vc = h->ext_v; e.qc = h->ext_q;
    e.rows_k = h->ext_rows_k; e.rows_q = (a->chunk_len + 127) / 128 * 128;
    e.stamps = h->base.stamps ? h->base.phase_ts : nullptr;
    e.sel_slots = h->base.sel_slots; e.sel_count = h->base.sel_count; e.attn_cs = h->base.attn_cs;
    e.err = h->base.err;
    e.wait_cycles = h->wait_cycles;

    // the selection kernel sees a batch of one request whose query is the fingerprint
    ts_decode_args d;
    memset(&d, 0, sizeof(d));
    d.struct_size = sizeof(d);
    d.layer = a->layer; d.batch = 1;
    d.q = h->ext_fp;
    d.k_pool = a->k_pool; d.v_pool = a->v_pool; d.pool_rows = a->pool_rows;
    d.req_to_token = a->req_to_token; d.req_to_token_stride = a->req_to_token_stride;
    d.req_pool_indices = h->ext_meta + 1; d.seq_lens = h->ext_meta;
    d.out = a->out;
    d.dbg_sel_slots = a->dbg_sel_slots; d.dbg_sel_pos = a->dbg_sel_pos;
    d.dbg_sel_count = a->dbg_sel_count; d.dbg_flags = a->dbg_flags;
    d.stream = a->stream;
    LayerParams p; Launch l;
    int s = fill(h, &d, p, l, fused_tp);
    if (s != TS_OK) return s;
    p.q_prerot = 1;
    p.attn_inline = 0;                   // the chunk's causal attention has kernels of its own
    TS_TRY(launch_extend_prep(e, l), "extend prepare");
    TS_TRY(launch_fused(p, l, fused_tp ? kModeTpFused : kModeAll), "select");
    TS_TRY(launch_extend_attend(e, l), "extend attend");
    if (a->dbg_fingerprint)
        TS_TRY(cudaMemcpyAsync(a->dbg_fingerprint, h->ext_fp, (size_t)c.hq * c.head_dim * h->elem,
                               cudaMemcpyDeviceToDevice, l.stream), "debug copy");
    return copy_debug(h, &d, p, l.stream);
}

int ts_get_counters(ts_handle* h, int32_t req_slot, uint64_t* retrievals, uint64_t* reuses, void* stream) {
    if (!h || req_slot < 0 || req_slot >= h->cfg.max_reqs) return TS_ERR_INVALID_ARG;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    unsigned long long v[2];
    TS_TRY(cudaMemcpyAsync(v, h->base.counters + 2 * (size_t)req_slot, 16, cudaMemcpyDeviceToHost, s), "counters");
    TS_TRY(cudaStreamSynchronize(s), "counters sync");
    if (retrievals) *retrievals = v[0];
    if (reuses) *reuses = v[1];
    return TS_OK;
}

int ts_last_error(ts_handle* h, int32_t* code, int32_t* detail) {
    if (!h) return TS_ERR_INVALID_ARG;
    int v[2] = {0, 0};
    TS_TRY(cudaDeviceSynchronize(), "sync");
    TS_TRY(cudaMemcpy(v, h->base.err, 8, cudaMemcpyDeviceToHost), "read error word");
    if (v[0] != 0) {
        TS_TRY(cudaMemset(h->base.err, 0, 8), "clear error word");
        // a grid barrier that gave up may have left its word mid-count
        TS_TRY(cudaMemset(h->base.grid_bar, 0, 4), "reset barrier word");
    }
    if (code) *code = v[0];
    if (detail) *detail = v[1];
    return TS_OK;
}

const char* ts_last_cuda_error(ts_handle* h) { return h ? h->cuda_msg : ""; }

int ts_debug_read(ts_handle* h, int32_t which, void* host_dst, size_t bytes) {
    if (!h || !host_dst) return TS_ERR_INVALID_ARG;
    const LayerParams& p = h->base;
    const void* src = nullptr;
    size_t avail = 0;
    const size_t hd = (size_t)h->cfg.hq * h->cfg.head_dim;
    switch (which) {
        case 0: src = p.q_rot; avail = (size_t)h->cfg.max_batch * hd * h->elem; break;
        case 1: src = p.logits; avail = (size_t)h->cand_capacity * h->cfg.hq * 4; break;
        case 2: src = p.votes_sel; avail = (size_t)h->cand_capacity * 4; break;
        case 3: src = p.phase_ts; avail = 128 * 8; break;
        case 4: src = p.cand_count; avail = (size_t)h->cfg.max_batch * 4; break;
        default: return TS_ERR_INVALID_ARG;
    }
    if (bytes > avail) return TS_ERR_INVALID_ARG;
    TS_TRY(cudaDeviceSynchronize(), "sync");
    TS_TRY(cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost), "debug read");
    return TS_OK;
}

int ts_timing_begin(ts_handle* h, int32_t max_launches) {
    if (!h || max_launches < 1) return TS_ERR_INVALID_ARG;
    if (h->timer.capacity < max_launches) {
        free_timer(h);
        h->timer.events = new (std::nothrow) cudaEvent_t[2 * (size_t)max_launches];
        h->timer.stages = new (std::nothrow) int[max_launches];
        if (!h->timer.events || !h->timer.stages) return TS_ERR_CUDA;
        for (int i = 0; i < 2 * max_launches; ++i) TS_TRY(cudaEventCreate(&h->timer.events[i]), "event create");
        h->timer.capacity = max_launches;
    }
    h->timer.used = 0;
    h->timer.on = 1;
    return TS_OK;
}

int ts_timing_end(ts_handle* h, double* ms_by_stage, uint64_t* launches_by_stage) {
    if (!h || !ms_by_stage || !launches_by_stage) return TS_ERR_INVALID_ARG;
    h->timer.on = 0;
    TS_TRY(cudaDeviceSynchronize(), "sync");
    for (int s = 0; s < TS_NUM_STAGES; ++s) { ms_by_stage[s] = 0.0; launches_by_stage[s] = 0; }
    for (int i = 0; i < h->timer.used; ++i) {
        float ms = 0.f;
        TS_TRY(cudaEventElapsedTime(&ms, h->timer.events[2 * i], h->timer.events[2 * i + 1]), "elapsed");
        const int s = h->timer.stages[i];
        if (s >= 0 && s < TS_NUM_STAGES) { ms_by_stage[s] += ms; ++launches_by_stage[s]; }
    }
    h->timer.used = 0;
    return TS_OK;
}

int ts_launch_count(ts_handle* h, uint64_t* launches) {
    if (!h || !launches) return TS_ERR_INVALID_ARG;
    *launches = h->launches;
    return TS_OK;
}

}  // extern "C"
