// One chunk of a prefill (at most 512 tokens) of one request, one layer: K/V rows of the chunk into the
// pools, the chunk's scoring query ("fingerprint"), selection by the same cooperative kernel as a decode
// step, then causal attention of the chunk's queries over the selected list.
//
// Replaces patched_radix_attention_extend_forward_flashinfer (token_retrieval.py:703-775) for one
// iteration of its chunk loop: store_kv_cache(start, end) (:726-734, :844-854), retrieval_indices with
// position_ids = arange(n_local, n_local + Lq) and torch.mean over the chunk (:380-392), the fall-back to
// all tokens (:741-744), and the paged prefill wrapper's causal forward with rotation on list positions
// (:746-772).  The per-chunk, per-layer host re-planning of that wrapper (:746-758) has no counterpart:
// the kernels read the selected list where the selection kernel left it.
//
// Launches: extend_prep_kernel -> fused_select_kernel (query pre-rotated) -> extend_gather_kernel ->
// extend_attend_tc_kernel (bf16, head_dim 128) or extend_attend_plain_kernel.
//
// The gather kernel writes the listed K rows, rotated at their list position and rounded to the model
// dtype, the listed V rows and the chunk's rotated queries into compact per-head arrays.  For the
// tensor-core kernel the 16-byte pieces of every 256-byte row are stored XOR-swizzled with the row number,
// so that a whole 64-row tile arrives with ONE bulk copy and ldmatrix reads it without bank conflicts.
#include <math.h>

#include "ptx.cuh"

namespace ts {

namespace {

constexpr int kExtThreads = 256;
constexpr int kTile = 64;                 // queries per CTA and keys per block of the tensor-core kernel
constexpr float kLog2eX = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ size_t swz(size_t row_base_elems, int row, int e, bool swizzle) {
    if (!swizzle) return row_base_elems + e;
    constexpr int per = 16 / (int)sizeof(T);               // elements per 16-byte piece
    const int piece = e / per, within = e - piece * per;
    return row_base_elems + (size_t)((piece ^ (row & 7)) * per + within);
}

// ------------------------------------------------------------------------------------------------
// 1. K/V rows of the chunk into the pools; fingerprint; the (length, request) pair the selection kernel reads
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kExtThreads) extend_prep_kernel(const ExtendParams e) {
    if (*(volatile int*)e.err != 0) return;
    const int half = e.d / 2, hd = e.hq * e.d;
    const int fp_blocks = (e.hq * half + kExtThreads - 1) / kExtThreads;
    const int lq = e.chunk_len;
    if (blockIdx.x == 0 && threadIdx.x == 0) { e.meta[0] = e.seq_len; e.meta[1] = e.req; }
    if ((int)blockIdx.x < fp_blocks) {
        // Pair (h, i): every query of the chunk rotated at position (n_local + t) * rope_scale and rounded
        // to the model dtype (:98-107), summed in fp32 in ascending t, divided once, rounded once.
        const int pidx = blockIdx.x * kExtThreads + threadIdx.x;
        if (pidx >= e.hq * half) return;
        const int h = pidx / half, i = pidx - h * half;
        const T* q = reinterpret_cast<const T*>(e.q) + (size_t)h * e.d + i;
        const float inv = (float)(1.0 / pow(e.rope_base, (double)(2 * i) / (double)e.d));
        float acc1 = 0.f, acc2 = 0.f;
#pragma unroll 4
        for (int t = 0; t < lq; ++t) {
            const float x1 = to_f32<T>(q[(size_t)t * hd]);
            const float x2 = to_f32<T>(q[(size_t)t * hd + half]);
            float2 cs;
            if (e.chunk_cs != nullptr) {
                cs = e.chunk_cs[(size_t)t * half + i];
            } else {
                const float ang = __fmul_rn((float)((double)(e.n_local + t) * e.rope_scale), inv);
                cs = make_float2(cosf(ang), sinf(ang));
            }
            const float r1 = __fadd_rn(__fmul_rn(x1, cs.x), __fmul_rn(-x2, cs.y));
            const float r2 = __fadd_rn(__fmul_rn(x2, cs.x), __fmul_rn(x1, cs.y));
            acc1 = __fadd_rn(acc1, to_f32<T>(from_f32<T>(r1)));
            acc2 = __fadd_rn(acc2, to_f32<T>(from_f32<T>(r2)));
        }
        T* fp = reinterpret_cast<T*>(e.fp) + (size_t)h * e.d + i;
        fp[0] = from_f32<T>(__fdiv_rn(acc1, (float)lq));
        fp[half] = from_f32<T>(__fdiv_rn(acc2, (float)lq));
        return;
    }
    if (e.k_new == nullptr) return;
    // append: row t of the chunk goes to pool row out_cache_loc[t]
    const int row_vec = e.hkv * e.d * (int)sizeof(T) / 16;
    const int nblk = gridDim.x - fp_blocks;
    for (int idx = (blockIdx.x - fp_blocks) * kExtThreads + threadIdx.x; idx < lq * row_vec; idx += nblk * kExtThreads) {
        const int t = idx / row_vec, c = idx - t * row_vec;
        const int loc = e.out_cache_loc[t];
        if (loc < 0 || loc >= e.pool_rows) { set_error(e.err, TS_ERR_BAD_SLOT, loc); continue; }
        reinterpret_cast<uint4*>(e.k_pool)[(size_t)loc * row_vec + c] = reinterpret_cast<const uint4*>(e.k_new)[idx];
        reinterpret_cast<uint4*>(e.v_pool)[(size_t)loc * row_vec + c] = reinterpret_cast<const uint4*>(e.v_new)[idx];
    }
}

// ------------------------------------------------------------------------------------------------
// 3. compact arrays: kc, vc [hkv][rows_k][d], qc [hq][rows_q][d]; rows beyond the list / the chunk are zero
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kExtThreads) extend_gather_kernel(const ExtendParams e, const int swizzle) {
    if (*(volatile int*)e.err != 0) return;
    const int half = e.d / 2;
    const int per_block = kExtThreads / half;
    const int item = blockIdx.x * per_block + threadIdx.x / half;
    const int i = threadIdx.x % half;
    const int count = min(*e.sel_count, e.n_sel);
    const int lq = e.chunk_len;
    const int k_items = e.rows_k * e.hkv;
    if (item < k_items) {
        const int j = item / e.hkv, kv = item - j * e.hkv;
        float r1 = 0.f, r2 = 0.f, v1 = 0.f, v2 = 0.f;
        if (j < count) {
            int slot = e.sel_slots[j];
            if ((unsigned long long)(long long)slot >= (unsigned long long)e.pool_rows) {
                set_error(e.err, TS_ERR_BAD_SLOT, slot);
                slot = 0;
            }
            const T* kr = reinterpret_cast<const T*>(e.k_pool) + ((size_t)slot * e.hkv + kv) * e.d;
            const T* vr = reinterpret_cast<const T*>(e.v_pool) + ((size_t)slot * e.hkv + kv) * e.d;
            const float x1 = to_f32<T>(kr[i]), x2 = to_f32<T>(kr[i + half]);
            const float2 cs = e.attn_cs[(size_t)j * half + i];          // list position j (:820-822)
            r1 = x1 * cs.x - x2 * cs.y;
            r2 = x2 * cs.x + x1 * cs.y;
            v1 = to_f32<T>(vr[i]);
            v2 = to_f32<T>(vr[i + half]);
        }
        const size_t base = ((size_t)kv * e.rows_k + j) * e.d;
        T* kc = reinterpret_cast<T*>(e.kc);
        T* vc = reinterpret_cast<T*>(e.vc);
        kc[swz<T>(base, j, i, swizzle)] = from_f32<T>(r1);
        kc[swz<T>(base, j, i + half, swizzle)] = from_f32<T>(r2);
        vc[swz<T>(base, j, i, swizzle)] = from_f32<T>(v1);
        vc[swz<T>(base, j, i + half, swizzle)] = from_f32<T>(v2);
        return;
    }
    const int qitem = item - k_items;
    if (qitem >= e.rows_q * e.hq) return;
    const int t = qitem / e.hq, h = qitem - t * e.hq;
    float r1 = 0.f, r2 = 0.f;
    if (t < lq) {
        const int pos = count - lq + t;                                   // the chunk closes the list
        const T* qr = reinterpret_cast<const T*>(e.q) + ((size_t)t * e.hq + h) * e.d;
        const float x1 = to_f32<T>(qr[i]), x2 = to_f32<T>(qr[i + half]);
        const float2 cs = e.attn_cs[(size_t)max(pos, 0) * half + i];
        r1 = x1 * cs.x - x2 * cs.y;
        r2 = x2 * cs.x + x1 * cs.y;
    }
    const size_t base = ((size_t)h * e.rows_q + t) * e.d;
    T* qc = reinterpret_cast<T*>(e.qc);
    qc[swz<T>(base, t, i, swizzle)] = from_f32<T>(r1);
    qc[swz<T>(base, t, i + half, swizzle)] = from_f32<T>(r2);
}

// ------------------------------------------------------------------------------------------------
// 4a. causal attention on the compact arrays, tensor cores (bf16, head_dim 128)
// ------------------------------------------------------------------------------------------------
// grid (rows_q / 64, hq), 128 threads.  Warp w owns query rows 16w..16w+15 of the tile; keys in blocks of 64,
// two stages, each block's K and V tile (16 KB each, contiguous in the compact arrays) fetched by one bulk
// copy.  S = Q K^T and O += P V with mma.sync m16n8k16 (bf16 in, fp32 accumulate), softmax in base 2.
struct ExtSmem {
    unsigned char q[kTile * 256];
    unsigned char k[2][kTile * 256];
    unsigned char v[2][kTile * 256];
    uint64_t qbar, full[2];
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(128, 2) extend_attend_tc_kernel(const ExtendParams e) {
    extern __shared__ __align__(128) unsigned char ext_dyn[];
    ExtSmem& sm = *reinterpret_cast<ExtSmem*>(ext_dyn);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int qt = blockIdx.x, h = blockIdx.y, kv = h / e.group;
    const int lq = e.chunk_len;
    if (*(volatile int*)e.err != 0 || qt * kTile >= lq) return;
    const int count = min(*e.sel_count, e.n_sel);
    const int base_vis = count - lq;                         // query row r sees list entries j <= base_vis + r
    const int kmax = min(count - 1, base_vis + qt * kTile + kTile - 1);
    const int nblk = kmax / kTile + 1;
    bool dead = false;

    const __nv_bfloat16* qsrc = reinterpret_cast<const __nv_bfloat16*>(e.qc) + ((size_t)h * e.rows_q + (size_t)qt * kTile) * 128;
    const __nv_bfloat16* ksrc = reinterpret_cast<const __nv_bfloat16*>(e.kc) + (size_t)kv * e.rows_k * 128;
    const __nv_bfloat16* vsrc = reinterpret_cast<const __nv_bfloat16*>(e.vc) + (size_t)kv * e.rows_k * 128;
    if (tid == 0) {
        mbar_init(smem_u32(&sm.qbar), 1);
        mbar_init(smem_u32(&sm.full[0]), 1);
        mbar_init(smem_u32(&sm.full[1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(smem_u32(&sm.qbar), kTile * 256);
        bulk_g2s(smem_u32(sm.q), qsrc, kTile * 256, smem_u32(&sm.qbar));
        for (int s = 0; s < 2 && s < nblk; ++s) {
            mbar_expect_tx(smem_u32(&sm.full[s]), 2 * kTile * 256);
            bulk_g2s(smem_u32(sm.k[s]), ksrc + (size_t)s * kTile * 128, kTile * 256, smem_u32(&sm.full[s]));
            bulk_g2s(smem_u32(sm.v[s]), vsrc + (size_t)s * kTile * 128, kTile * 256, smem_u32(&sm.full[s]));
        }
    }
    __syncthreads();

    // query fragments: 8 k-steps of 16
    uint32_t qa[8][4];
    mbar_wait(smem_u32(&sm.qbar), 0, e.err, dead, 40);
    {
        const int row = warp * 16 + (lane & 15);
        const uint32_t rbase = smem_u32(sm.q) + row * 256;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int piece = 2 * ks + (lane >> 4);
            ldmatrix_x4(qa[ks], rbase + ((piece ^ (row & 7)) << 4));
        }
    }
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] = 0.f; o[n][1] = 0.f; o[n][2] = 0.f; o[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row0 = qt * kTile + warp * 16 + g;
    const int lim0 = base_vis + row0, lim1 = lim0 + 8;
    const float scale = e.sm_scale;
    const float cap = e.logit_cap;

    for (int blk = 0; blk < nblk; ++blk) {
        const int s = blk & 1;
        mbar_wait(smem_u32(&sm.full[s]), (uint32_t)((blk >> 1) & 1), e.err, dead, 41);
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { sc[n][0] = 0.f; sc[n][1] = 0.f; sc[n][2] = 0.f; sc[n][3] = 0.f; }
        const uint32_t kb = smem_u32(sm.k[s]);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const int row = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int piece = 2 * ks + ((lane >> 3) & 1);
                uint32_t b[4];
                ldmatrix_x4(b, kb + row * 256 + ((piece ^ (row & 7)) << 4));
                mma_bf16_16816(sc[2 * np], qa[ks], b[0], b[1]);
                mma_bf16_16816(sc[2 * np + 1], qa[ks], b[2], b[3]);
            }
        }
        // scale, soft cap, causal mask, base-2 units
        const int key0 = blk * kTile + 2 * t4;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float x = sc[n][c] * scale;
                if (cap > 0.f) x = cap * tanhf(x / cap);
                x *= kLog2eX;
                const int key = key0 + n * 8 + (c & 1);
                const int lim = (c < 2) ? lim0 : lim1;
                if (key > lim) x = -INFINITY;
                sc[n][c] = x;
            }
            mx0 = fmaxf(mx0, fmaxf(sc[n][0], sc[n][1]));
            mx1 = fmaxf(mx1, fmaxf(sc[n][2], sc[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        // a row whose every entry so far is masked keeps (max, sum) = (-inf, 0) and contributes nothing
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = exp2f(m_run[0] - ref0), corr1 = exp2f(m_run[1] - ref1);
        m_run[0] = mn0; m_run[1] = mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            sc[n][0] = exp2f(sc[n][0] - ref0); sc[n][1] = exp2f(sc[n][1] - ref0);
            sc[n][2] = exp2f(sc[n][2] - ref1); sc[n][3] = exp2f(sc[n][3] - ref1);
            sum0 += sc[n][0] + sc[n][1];
            sum1 += sc[n][2] + sc[n][3];
        }
        l_run[0] = l_run[0] * corr0 + sum0;
        l_run[1] = l_run[1] * corr1 + sum1;
#pragma unroll
        for (int n = 0; n < 16; ++n) { o[n][0] *= corr0; o[n][1] *= corr0; o[n][2] *= corr1; o[n][3] *= corr1; }
        // O += P V
        const uint32_t vb = smem_u32(sm.v[s]);
#pragma unroll
        for (int kb16 = 0; kb16 < 4; ++kb16) {
            uint32_t a[4];
            a[0] = pack_bf16(sc[2 * kb16][0], sc[2 * kb16][1]);
            a[1] = pack_bf16(sc[2 * kb16][2], sc[2 * kb16][3]);
            a[2] = pack_bf16(sc[2 * kb16 + 1][0], sc[2 * kb16 + 1][1]);
            a[3] = pack_bf16(sc[2 * kb16 + 1][2], sc[2 * kb16 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {
                const int row = kb16 * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int piece = 2 * dp + (lane >> 4);
                uint32_t b[4];
                ldmatrix_x4_trans(b, vb + row * 256 + ((piece ^ (row & 7)) << 4));
                mma_bf16_16816(o[2 * dp], a, b[0], b[1]);
                mma_bf16_16816(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();                                    // every warp is done with stage s
        if (tid == 0 && blk + 2 < nblk) {
            asm volatile("fence.proxy.async;" ::: "memory");
            mbar_expect_tx(smem_u32(&sm.full[s]), 2 * kTile * 256);
            bulk_g2s(smem_u32(sm.k[s]), ksrc + (size_t)(blk + 2) * kTile * 128, kTile * 256, smem_u32(&sm.full[s]));
            bulk_g2s(smem_u32(sm.v[s]), vsrc + (size_t)(blk + 2) * kTile * 128, kTile * 256, smem_u32(&sm.full[s]));
        }
    }
    // the row sums were kept per thread: join the four threads of a row
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(e.out);
    const size_t hd = (size_t)e.hq * 128;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
        const int col = h * 128 + n * 8 + 2 * t4;
        if (row0 < lq)
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row0 * hd + col) = __floats2bfloat162_rn(o[n][0] * inv0, o[n][1] * inv0);
        if (row0 + 8 < lq)
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(row0 + 8) * hd + col) = __floats2bfloat162_rn(o[n][2] * inv1, o[n][3] * inv1);
    }
}

// ------------------------------------------------------------------------------------------------
// 4b. the same on CUDA cores in fp32 (fp32 check mode, head_dim 64): one warp per (query, head)
// ------------------------------------------------------------------------------------------------
template <typename T, int E>
__global__ void __launch_bounds__(kExtThreads) extend_attend_plain_kernel(const ExtendParams e) {
    constexpr int D = 32 * E;
    if (*(volatile int*)e.err != 0) return;
    const int lane = threadIdx.x & 31;
    const int w = blockIdx.x * (kExtThreads / 32) + (threadIdx.x >> 5);
    const int lq = e.chunk_len;
    if (w >= lq * e.hq) return;
    const int t = w / e.hq, h = w - t * e.hq, kv = h / e.group;
    const int count = min(*e.sel_count, e.n_sel);
    const int lim = count - lq + t;
    const T* qr = reinterpret_cast<const T*>(e.qc) + ((size_t)h * e.rows_q + t) * D;
    const T* kc = reinterpret_cast<const T*>(e.kc) + (size_t)kv * e.rows_k * D;
    const T* vc = reinterpret_cast<const T*>(e.vc) + (size_t)kv * e.rows_k * D;
    float q[E], acc[E];
#pragma unroll
    for (int x = 0; x < E; ++x) { q[x] = to_f32<T>(qr[lane + 32 * x]); acc[x] = 0.f; }
    float m = -INFINITY, l = 0.f;
    for (int j = 0; j <= lim; ++j) {
        float s = 0.f;
#pragma unroll
        for (int x = 0; x < E; ++x) s += q[x] * to_f32<T>(kc[(size_t)j * D + lane + 32 * x]);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        float x = s * e.sm_scale;
        if (e.logit_cap > 0.f) x = e.logit_cap * tanhf(x / e.logit_cap);
        x *= kLog2eX;
        const float mn = fmaxf(m, x);
        const float corr = exp2f(m - mn), pe = exp2f(x - mn);
        l = l * corr + pe;
        m = mn;
#pragma unroll
        for (int y = 0; y < E; ++y) acc[y] = acc[y] * corr + pe * to_f32<T>(vc[(size_t)j * D + lane + 32 * y]);
    }
    T* out = reinterpret_cast<T*>(e.out) + ((size_t)t * e.hq + h) * D;
#pragma unroll
    for (int x = 0; x < E; ++x) out[lane + 32 * x] = from_f32<T>(acc[x] / l);
}

template <typename T>
cudaError_t launch_extend_prep_t(const ExtendParams& e, const Launch& l) {
    const int half = e.d / 2;
    const int fp_blocks = (e.hq * half + kExtThreads - 1) / kExtThreads;
    const int row_vec = e.hkv * e.d * (int)sizeof(T) / 16;
    int app = e.k_new ? (e.chunk_len * row_vec + kExtThreads - 1) / kExtThreads : 0;
    if (app > 4 * l.num_sms) app = 4 * l.num_sms;
    stage_begin(l, kStageExtendPrep);
    extend_prep_kernel<T><<<fp_blocks + app, kExtThreads, 0, l.stream>>>(e);
    stage_end(l);
    return cudaGetLastError();
}

}  // namespace

bool extend_uses_tensor_cores(int dtype, int d, int group) {
    return dtype == TS_DTYPE_BF16 && d == 128 && group >= 1;
}

cudaError_t launch_extend_prep(const ExtendParams& e, const Launch& l) {
    return l.dtype == TS_DTYPE_BF16 ? launch_extend_prep_t<__nv_bfloat16>(e, l) : launch_extend_prep_t<float>(e, l);
}

cudaError_t launch_extend_attend(const ExtendParams& e, const Launch& l) {
    const bool tc = extend_uses_tensor_cores(l.dtype, e.d, e.group);
    const int half = e.d / 2;
    const int items = e.rows_k * e.hkv + e.rows_q * e.hq;
    const int per_block = kExtThreads / half;
    stage_begin(l, kStageExtendGather);
    if (l.dtype == TS_DTYPE_BF16)
        extend_gather_kernel<__nv_bfloat16><<<(items + per_block - 1) / per_block, kExtThreads, 0, l.stream>>>(e, tc ? 1 : 0);
    else
        extend_gather_kernel<float><<<(items + per_block - 1) / per_block, kExtThreads, 0, l.stream>>>(e, 0);
    stage_end(l);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    stage_begin(l, kStageExtendAttend);
    if (tc) {
        static bool configured = false;
        if (!configured) {
            err = cudaFuncSetAttribute(extend_attend_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ExtSmem));
            if (err != cudaSuccess) return err;
            configured = true;
        }
        extend_attend_tc_kernel<<<dim3(e.rows_q / kTile, e.hq), 128, sizeof(ExtSmem), l.stream>>>(e);
    } else {
        const int warps = e.chunk_len * e.hq;
        const int blocks = (warps + kExtThreads / 32 - 1) / (kExtThreads / 32);
        if (l.dtype == TS_DTYPE_BF16) {
            if (e.d == 128) extend_attend_plain_kernel<__nv_bfloat16, 4><<<blocks, kExtThreads, 0, l.stream>>>(e);
            else extend_attend_plain_kernel<__nv_bfloat16, 2><<<blocks, kExtThreads, 0, l.stream>>>(e);
        } else {
            if (e.d == 128) extend_attend_plain_kernel<float, 4><<<blocks, kExtThreads, 0, l.stream>>>(e);
            else extend_attend_plain_kernel<float, 2><<<blocks, kExtThreads, 0, l.stream>>>(e);
        }
    }
    stage_end(l);
    return cudaGetLastError();
}

}  // namespace ts
