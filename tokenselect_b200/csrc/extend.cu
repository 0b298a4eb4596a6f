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
constexpr int kTile = 64;                 // keys per block of the tensor-core kernel
constexpr float kLog2eX = 1.4426950408889634f;

// ------------------------------------------------------------------------------------------------
// 1. K/V rows of the chunk into the pools; fingerprint; the (length, request) pair the selection kernel reads
// ------------------------------------------------------------------------------------------------
// Fingerprint: four warps own eight adjacent rotation pairs (h, i0..i0+7).  Every query t is rotated at position
// (n_local + t) * rope_scale and rounded to the model dtype (:98-107).  Summation order (torch.mean leaves
// it open; this one is fixed): 128 fp32 partial sums, partial s taking t = s, s+128, ... in ascending order;
// lane j joins its four partials ((j + (j+32)) + (j+64)) + (j+96); an XOR butterfly (16, 8, 4, 2, 1) joins
// the lanes; one fp32 division by the chunk length, one rounding.
template <typename T>
__global__ void __launch_bounds__(kExtThreads) extend_prep_kernel(const ExtendParams e) {
    __shared__ float part[2][4][32][16];
    if (*(volatile int*)e.err != 0) return;
    const int half = e.d / 2, hd = e.hq * e.d;
    const int groups = e.hq * half / 8;                                   // groups of eight pairs
    const int fp_blocks = (groups + 1) / 2;                               // two groups per CTA, four warps each
    const int lq = e.chunk_len;
    if (blockIdx.x == 0 && threadIdx.x == 0) { e.meta[0] = e.seq_len; e.meta[1] = e.req; }
    if ((int)blockIdx.x < fp_blocks) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int gl = warp >> 2, c = warp & 3;                           // group inside the CTA, chain of this warp
        const int grp = min(blockIdx.x * 2 + gl, groups - 1);
        const bool live = (int)blockIdx.x * 2 + gl < groups;
        const int h = grp / (half / 8), i0 = (grp - h * (half / 8)) * 8;
        const T* q = reinterpret_cast<const T*>(e.q) + (size_t)h * e.d + i0;
        float inv[8];
        if (e.chunk_cs == nullptr) {
#pragma unroll
            for (int u = 0; u < 8; ++u) inv[u] = (float)(1.0 / pow(e.rope_base, (double)(2 * (i0 + u)) / (double)e.d));
        }
        // warp c of a group holds partial sums s = lane + 32c: queries t = s, s+128, ... in ascending order
        float a1[8], a2[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) { a1[u] = 0.f; a2[u] = 0.f; }
#pragma unroll 4
        for (int t = lane + 32 * c; t < lq; t += 128) {
            T x1[8], x2[8];
            if constexpr (sizeof(T) == 2) {
                *reinterpret_cast<uint4*>(x1) = *reinterpret_cast<const uint4*>(q + (size_t)t * hd);
                *reinterpret_cast<uint4*>(x2) = *reinterpret_cast<const uint4*>(q + (size_t)t * hd + half);
            } else {
#pragma unroll
                for (int u = 0; u < 8; u += 4) {
                    *reinterpret_cast<float4*>(x1 + u) = *reinterpret_cast<const float4*>(q + (size_t)t * hd + u);
                    *reinterpret_cast<float4*>(x2 + u) = *reinterpret_cast<const float4*>(q + (size_t)t * hd + half + u);
                }
            }
            float2 cs[8];
            if (e.chunk_cs != nullptr) {
                const float4* src = reinterpret_cast<const float4*>(e.chunk_cs + (size_t)t * half + i0);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float4 v = src[u];
                    cs[2 * u] = make_float2(v.x, v.y);
                    cs[2 * u + 1] = make_float2(v.z, v.w);
                }
            } else {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float ang = __fmul_rn((float)((double)(e.n_local + t) * e.rope_scale), inv[u]);
                    cs[u] = make_float2(cosf(ang), sinf(ang));
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float xa = to_f32<T>(x1[u]), xb = to_f32<T>(x2[u]);
                const float r1 = __fadd_rn(__fmul_rn(xa, cs[u].x), __fmul_rn(-xb, cs[u].y));
                const float r2 = __fadd_rn(__fmul_rn(xb, cs[u].x), __fmul_rn(xa, cs[u].y));
                a1[u] = __fadd_rn(a1[u], to_f32<T>(from_f32<T>(r1)));
                a2[u] = __fadd_rn(a2[u], to_f32<T>(from_f32<T>(r2)));
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) { part[gl][c][lane][u] = a1[u]; part[gl][c][lane][8 + u] = a2[u]; }
        __syncthreads();
        if (c != 0 || !live) return;
        float acc1[8], acc2[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            acc1[u] = __fadd_rn(__fadd_rn(__fadd_rn(part[gl][0][lane][u], part[gl][1][lane][u]), part[gl][2][lane][u]),
                                part[gl][3][lane][u]);
            acc2[u] = __fadd_rn(__fadd_rn(__fadd_rn(part[gl][0][lane][8 + u], part[gl][1][lane][8 + u]),
                                          part[gl][2][lane][8 + u]), part[gl][3][lane][8 + u]);
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                acc1[u] = __fadd_rn(acc1[u], __shfl_xor_sync(0xffffffffu, acc1[u], o));
                acc2[u] = __fadd_rn(acc2[u], __shfl_xor_sync(0xffffffffu, acc2[u], o));
            }
        }
        if (lane == 0) {
            T* fp = reinterpret_cast<T*>(e.fp) + (size_t)h * e.d + i0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                fp[u] = from_f32<T>(__fdiv_rn(acc1[u], (float)lq));
                fp[half + u] = from_f32<T>(__fdiv_rn(acc2[u], (float)lq));
            }
        }
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
// A thread owns eight adjacent rotation pairs of one (row, head): elements i0..i0+7 of both halves, i.e.
// one 16-byte piece per half in bf16.
template <typename T>
__device__ __forceinline__ void load8(const T* src, float (&x)[8]) {
    if constexpr (sizeof(T) == 2) {
        T raw[8];
        *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(src);
#pragma unroll
        for (int u = 0; u < 8; ++u) x[u] = to_f32<T>(raw[u]);
    } else {
#pragma unroll
        for (int u = 0; u < 8; u += 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + u);
            x[u] = v.x; x[u + 1] = v.y; x[u + 2] = v.z; x[u + 3] = v.w;
        }
    }
}
// Layouts of the compact arrays (per head: `rows` rows of d elements):
//   kLayoutPlain   row-major;
//   kLayoutXor16   row-major, the sixteen 16-byte pieces of a 256-byte row XOR-ed with row & 7 (mma.sync kernel);
//   kLayoutImage   tiles of `tile_rows` rows stored as the shared-memory image tcgen05 reads: per tile the
//                  two 64-element halves one after the other, each [row][128 B] with the eight 16-byte
//                  pieces of a row XOR-ed with row & 7 (the 128-byte swizzle of the K-major / MN-major
//                  canonical layouts), so that one linear bulk copy brings a whole operand tile.
enum { kLayoutPlain = 0, kLayoutXor16 = 1, kLayoutImage = 2 };

template <typename T>
__device__ __forceinline__ void store8(T* head_base, int d, int row, int e0, const float (&x)[8], int layout, int tile_rows) {
    if constexpr (sizeof(T) == 2) {
        T raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) raw[u] = from_f32<T>(x[u]);
        size_t off;                                                        // in elements
        if (layout == kLayoutImage) {
            const int tile = row / tile_rows, r = row - tile * tile_rows;
            const int hlf = e0 >> 6, piece = (e0 & 63) >> 3;
            off = (size_t)tile * tile_rows * 128 + (size_t)hlf * tile_rows * 64 + (size_t)r * 64 + ((piece ^ (r & 7)) << 3);
        } else {
            const int piece = e0 >> 3;
            off = (size_t)row * d + ((layout == kLayoutXor16 ? (piece ^ (row & 7)) : piece) << 3);
        }
        *reinterpret_cast<uint4*>(head_base + off) = *reinterpret_cast<uint4*>(raw);
    } else {
#pragma unroll
        for (int u = 0; u < 8; u += 4)
            *reinterpret_cast<float4*>(head_base + (size_t)row * d + e0 + u) = make_float4(x[u], x[u + 1], x[u + 2], x[u + 3]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kExtThreads) extend_gather_kernel(const ExtendParams e, const int layout, const int kv_tile) {
    // the attention kernel that follows may be scheduled now: it waits (griddepcontrol.wait) for this grid to finish
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (*(volatile int*)e.err != 0) return;
    const int half = e.d / 2;
    const int tpi = half / 8;                                             // threads per (row, head) item
    const int per_block = kExtThreads / tpi;
    const int item = blockIdx.x * per_block + threadIdx.x / tpi;
    const int i0 = (threadIdx.x % tpi) * 8;
    const int count = min(*e.sel_count, e.n_sel);
    const int lq = e.chunk_len;
    const int k_items = e.rows_k * e.hkv;
    float z[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) z[u] = 0.f;
    if (item < k_items) {
        const int j = item / e.hkv, kv = item - j * e.hkv;
        T* kc = reinterpret_cast<T*>(e.kc) + (size_t)kv * e.rows_k * e.d;
        T* vc = reinterpret_cast<T*>(e.vc) + (size_t)kv * e.rows_k * e.d;
        if (j >= count) {
            store8<T>(kc, e.d, j, i0, z, layout, kv_tile); store8<T>(kc, e.d, j, i0 + half, z, layout, kv_tile);
            store8<T>(vc, e.d, j, i0, z, layout, kv_tile); store8<T>(vc, e.d, j, i0 + half, z, layout, kv_tile);
            return;
        }
        int slot = e.sel_slots[j];
        if ((unsigned long long)(long long)slot >= (unsigned long long)e.pool_rows) {
            set_error(e.err, TS_ERR_BAD_SLOT, slot);
            slot = 0;
        }
        const T* kr = reinterpret_cast<const T*>(e.k_pool) + ((size_t)slot * e.hkv + kv) * e.d;
        const T* vr = reinterpret_cast<const T*>(e.v_pool) + ((size_t)slot * e.hkv + kv) * e.d;
        float x1[8], x2[8], v1[8], v2[8], r1[8], r2[8];
        load8<T>(kr + i0, x1); load8<T>(kr + i0 + half, x2);
        load8<T>(vr + i0, v1); load8<T>(vr + i0 + half, v2);
        const float2* cs = e.attn_cs + (size_t)j * half + i0;            // list position j (:820-822)
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float2 c = cs[u];
            r1[u] = x1[u] * c.x - x2[u] * c.y;
            r2[u] = x2[u] * c.x + x1[u] * c.y;
        }
        store8<T>(kc, e.d, j, i0, r1, layout, kv_tile); store8<T>(kc, e.d, j, i0 + half, r2, layout, kv_tile);
        store8<T>(vc, e.d, j, i0, v1, layout, kv_tile); store8<T>(vc, e.d, j, i0 + half, v2, layout, kv_tile);
        return;
    }
    const int qitem = item - k_items;
    if (qitem >= e.rows_q * e.hq) return;
    const int t = qitem / e.hq, h = qitem - t * e.hq;
    T* qc = reinterpret_cast<T*>(e.qc) + (size_t)h * e.rows_q * e.d;
    if (t >= lq) {
        store8<T>(qc, e.d, t, i0, z, layout, 128); store8<T>(qc, e.d, t, i0 + half, z, layout, 128);
        return;
    }
    const int pos = max(count - lq + t, 0);                               // the chunk closes the list
    const T* qr = reinterpret_cast<const T*>(e.q) + ((size_t)t * e.hq + h) * e.d;
    float x1[8], x2[8], r1[8], r2[8];
    load8<T>(qr + i0, x1); load8<T>(qr + i0 + half, x2);
    const float2* cs = e.attn_cs + (size_t)pos * half + i0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const float2 c = cs[u];
        r1[u] = x1[u] * c.x - x2[u] * c.y;
        r2[u] = x2[u] * c.x + x1[u] * c.y;
    }
    store8<T>(qc, e.d, t, i0, r1, layout, 128); store8<T>(qc, e.d, t, i0 + half, r2, layout, 128);
}

// ------------------------------------------------------------------------------------------------
// 4a. causal attention on the compact arrays, tensor cores (bf16, head_dim 128)
// ------------------------------------------------------------------------------------------------
// grid (rows_q / 128, hq), 128 threads.  Warp w owns query rows 32w..32w+31 of the tile (two 16-row mma
// tiles, so every K / V fragment read from shared memory feeds two mma); keys in blocks of 64, two stages,
// each block's K and V tile (16 KB each, contiguous in the compact arrays) fetched by one bulk copy.
// S = Q K^T and O += P V with mma.sync m16n8k16 (bf16 in, fp32 accumulate), softmax in base 2.  The
// query fragments are re-read from shared memory in every block (registers hold the 32 x 128 output).
constexpr int kQTile = 128;
struct ExtSmem {
    unsigned char q[kQTile * 256];
    unsigned char k[2][kTile * 256];
    unsigned char v[2][kTile * 256];
    uint64_t qbar, full[2];
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(128, 1) extend_attend_tc_kernel(const ExtendParams e) {
    extern __shared__ __align__(128) unsigned char ext_dyn[];
    ExtSmem& sm = *reinterpret_cast<ExtSmem*>(ext_dyn);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int qt = blockIdx.x, h = blockIdx.y, kv = h / e.group;
    const int lq = e.chunk_len;
    if (*(volatile int*)e.err != 0 || qt * kQTile >= lq) return;
    const int count = min(*e.sel_count, e.n_sel);
    const int base_vis = count - lq;                         // query row r sees list entries j <= base_vis + r
    const int kmax = min(count - 1, base_vis + qt * kQTile + kQTile - 1);
    const int nblk = kmax / kTile + 1;
    bool dead = false;

    const __nv_bfloat16* qsrc = reinterpret_cast<const __nv_bfloat16*>(e.qc) + ((size_t)h * e.rows_q + (size_t)qt * kQTile) * 128;
    const __nv_bfloat16* ksrc = reinterpret_cast<const __nv_bfloat16*>(e.kc) + (size_t)kv * e.rows_k * 128;
    const __nv_bfloat16* vsrc = reinterpret_cast<const __nv_bfloat16*>(e.vc) + (size_t)kv * e.rows_k * 128;
    if (tid == 0) {
        mbar_init(smem_u32(&sm.qbar), 1);
        mbar_init(smem_u32(&sm.full[0]), 1);
        mbar_init(smem_u32(&sm.full[1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(smem_u32(&sm.qbar), kQTile * 256);
        bulk_g2s(smem_u32(sm.q), qsrc, kQTile * 256, smem_u32(&sm.qbar));
        for (int s = 0; s < 2 && s < nblk; ++s) {
            mbar_expect_tx(smem_u32(&sm.full[s]), 2 * kTile * 256);
            bulk_g2s(smem_u32(sm.k[s]), ksrc + (size_t)s * kTile * 128, kTile * 256, smem_u32(&sm.full[s]));
            bulk_g2s(smem_u32(sm.v[s]), vsrc + (size_t)s * kTile * 128, kTile * 256, smem_u32(&sm.full[s]));
        }
    }
    __syncthreads();
    mbar_wait(smem_u32(&sm.qbar), 0, e.err, dead, 40, e.wait_cycles);

    float o[2][16][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int n = 0; n < 16; ++n) { o[mt][n][0] = 0.f; o[mt][n][1] = 0.f; o[mt][n][2] = 0.f; o[mt][n][3] = 0.f; }
    float m_run[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, l_run[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    const int row_base = qt * kQTile + warp * 32;            // first query row of this warp
    const float scale = e.sm_scale;
    const float cap = e.logit_cap;
    // ldmatrix source of the query fragments: row of the 128-row tile, 16-byte piece selector
    const int qrow0 = warp * 32 + (lane & 15);
    const uint32_t qb0 = smem_u32(sm.q) + qrow0 * 256, qb1 = qb0 + 16 * 256;
    const int qsw = qrow0 & 7, qhi = lane >> 4;              // (row + 16) & 7 == row & 7

    for (int blk = 0; blk < nblk; ++blk) {
        const int s = blk & 1;
        mbar_wait(smem_u32(&sm.full[s]), (uint32_t)((blk >> 1) & 1), e.err, dead, 41, e.wait_cycles);
        float sc[2][8][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int n = 0; n < 8; ++n) { sc[mt][n][0] = 0.f; sc[mt][n][1] = 0.f; sc[mt][n][2] = 0.f; sc[mt][n][3] = 0.f; }
        const uint32_t kb = smem_u32(sm.k[s]);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t qa0[4], qa1[4];
            const int qpiece = ((2 * ks + qhi) ^ qsw) << 4;
            ldmatrix_x4(qa0, qb0 + qpiece);
            ldmatrix_x4(qa1, qb1 + qpiece);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const int row = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int piece = 2 * ks + ((lane >> 3) & 1);
                uint32_t b[4];
                ldmatrix_x4(b, kb + row * 256 + ((piece ^ (row & 7)) << 4));
                mma_bf16_16816(sc[0][2 * np], qa0, b[0], b[1]);
                mma_bf16_16816(sc[0][2 * np + 1], qa0, b[2], b[3]);
                mma_bf16_16816(sc[1][2 * np], qa1, b[0], b[1]);
                mma_bf16_16816(sc[1][2 * np + 1], qa1, b[2], b[3]);
            }
        }
        // scale, soft cap, causal mask, base-2 units; online softmax per row
        const int key0 = blk * kTile + 2 * t4;
        const bool need_mask = blk * kTile + kTile - 1 > base_vis + row_base;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const int lim0 = base_vis + row_base + mt * 16 + g, lim1 = lim0 + 8;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float x = sc[mt][n][c] * scale;
                    if (cap > 0.f) x = cap * tanhf(x / cap);
                    x *= kLog2eX;
                    if (need_mask) {
                        const int key = key0 + n * 8 + (c & 1);
                        if (key > ((c < 2) ? lim0 : lim1)) x = -INFINITY;
                    }
                    sc[mt][n][c] = x;
                }
                mx0 = fmaxf(mx0, fmaxf(sc[mt][n][0], sc[mt][n][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[mt][n][2], sc[mt][n][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m_run[mt][0], mx0), mn1 = fmaxf(m_run[mt][1], mx1);
            // a row whose every entry so far is masked keeps (max, sum) = (-inf, 0) and contributes nothing
            const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
            const float corr0 = exp2f(m_run[mt][0] - ref0), corr1 = exp2f(m_run[mt][1] - ref1);
            m_run[mt][0] = mn0; m_run[mt][1] = mn1;
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                sc[mt][n][0] = exp2f(sc[mt][n][0] - ref0); sc[mt][n][1] = exp2f(sc[mt][n][1] - ref0);
                sc[mt][n][2] = exp2f(sc[mt][n][2] - ref1); sc[mt][n][3] = exp2f(sc[mt][n][3] - ref1);
                sum0 += sc[mt][n][0] + sc[mt][n][1];
                sum1 += sc[mt][n][2] + sc[mt][n][3];
            }
            l_run[mt][0] = l_run[mt][0] * corr0 + sum0;
            l_run[mt][1] = l_run[mt][1] * corr1 + sum1;
#pragma unroll
            for (int n = 0; n < 16; ++n) { o[mt][n][0] *= corr0; o[mt][n][1] *= corr0; o[mt][n][2] *= corr1; o[mt][n][3] *= corr1; }
        }
        // O += P V
        const uint32_t vb = smem_u32(sm.v[s]);
#pragma unroll
        for (int kb16 = 0; kb16 < 4; ++kb16) {
            uint32_t a0[4], a1[4];
            a0[0] = pack_bf16(sc[0][2 * kb16][0], sc[0][2 * kb16][1]);
            a0[1] = pack_bf16(sc[0][2 * kb16][2], sc[0][2 * kb16][3]);
            a0[2] = pack_bf16(sc[0][2 * kb16 + 1][0], sc[0][2 * kb16 + 1][1]);
            a0[3] = pack_bf16(sc[0][2 * kb16 + 1][2], sc[0][2 * kb16 + 1][3]);
            a1[0] = pack_bf16(sc[1][2 * kb16][0], sc[1][2 * kb16][1]);
            a1[1] = pack_bf16(sc[1][2 * kb16][2], sc[1][2 * kb16][3]);
            a1[2] = pack_bf16(sc[1][2 * kb16 + 1][0], sc[1][2 * kb16 + 1][1]);
            a1[3] = pack_bf16(sc[1][2 * kb16 + 1][2], sc[1][2 * kb16 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {
                const int row = kb16 * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int piece = 2 * dp + (lane >> 4);
                uint32_t b[4];
                ldmatrix_x4_trans(b, vb + row * 256 + ((piece ^ (row & 7)) << 4));
                mma_bf16_16816(o[0][2 * dp], a0, b[0], b[1]);
                mma_bf16_16816(o[0][2 * dp + 1], a0, b[2], b[3]);
                mma_bf16_16816(o[1][2 * dp], a1, b[0], b[1]);
                mma_bf16_16816(o[1][2 * dp + 1], a1, b[2], b[3]);
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
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(e.out);
    const size_t hd = (size_t)e.hq * 128;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        // the row sums were kept per thread: join the four threads of a row
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[mt][r] += __shfl_xor_sync(0xffffffffu, l_run[mt][r], 1);
            l_run[mt][r] += __shfl_xor_sync(0xffffffffu, l_run[mt][r], 2);
        }
        const float inv0 = l_run[mt][0] > 0.f ? 1.f / l_run[mt][0] : 0.f;
        const float inv1 = l_run[mt][1] > 0.f ? 1.f / l_run[mt][1] : 0.f;
        const int row0 = row_base + mt * 16 + g;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            const int col = h * 128 + n * 8 + 2 * t4;
            if (row0 < lq)
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row0 * hd + col) =
                    __floats2bfloat162_rn(o[mt][n][0] * inv0, o[mt][n][1] * inv0);
            if (row0 + 8 < lq)
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(row0 + 8) * hd + col) =
                    __floats2bfloat162_rn(o[mt][n][2] * inv1, o[mt][n][3] * inv1);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// 4a'. the same with the 5th-generation tensor cores: tcgen05.mma, accumulators in tensor memory
// ------------------------------------------------------------------------------------------------
// grid (rows_q / 128, hq), 544 threads, one CTA per SM.  M = 128 query rows per CTA; keys in blocks of 64.
//   S[b&1] (128 x 64 fp32, TMEM columns 64*(b&1)..)  = Q (smem, K-major SW128) . K_b^T (smem, K-major SW128)
//   O      (128 x 128 fp32, TMEM columns 128..255)  += P_b (TMEM columns 256 + 32*(b&1).., packed bf16) . V_b (smem, MN-major SW128)
// Four threads share TMEM lane r == query row r (a quarter of the columns each): they read S with
// tcgen05.ld, keep the row's reference maximum and partial sums and write P = 2^(S - ref) back to tensor
// memory as bf16.  O stays in tensor memory across blocks; it is rescaled (tcgen05.ld / st) only when a
// row's maximum has grown by more than 2^8 since the reference was taken, so P never exceeds 256.  One
// thread of a separate warp issues the MMAs: Q.K^T of block b+1 is issued before the softmax of block b
// starts, so the tensor pipe works under the softmax.
// K/V tiles: four stages, one bulk copy each per tile (the gather kernel stores them as smem images).
constexpr int kKvStages = 4;
struct Tc5Smem {
    unsigned char q[128 * 256];                 // 2 halves x [128 rows][128 B]
    unsigned char k[kKvStages][kTile * 256];    // 2 halves x [64 keys][128 B]
    unsigned char v[kKvStages][kTile * 256];
    float rowmax[2][4][128];                    // [block parity][column quarter][row]: row maxima; row sums at the end
    uint64_t qbar, full[kKvStages], s_done[2], o_done[2], p_ready[2];
    uint32_t tmem_base;
};

__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // start address, leading / stride byte offsets in 16-byte units; descriptor version 1; 128-byte swizzle
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
// A operand in tensor memory (rows = lanes, two bf16 per 32-bit column), B through a shared-memory descriptor
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// 4 * NS softmax warps + 1 issuer warp (NS = 2 by default).  Softmax thread (column slice c = warp / 4, lane
// quarter w = warp % 4, lane l) owns query row 32w + l and the columns [64c/NS, 64(c+1)/NS) of S,
// [128c/NS, 128(c+1)/NS) of O; the NS threads of a row exchange the row maximum through shared memory (a named
// barrier per lane quarter) and keep separate partial sums.  P goes back to tensor memory as packed bf16 and is the A operand of P.V.
// Lane 0 of the issuer warp requests tiles and issues every MMA.
constexpr uint32_t kTmemCols = 512, kTmemO = 128, kTmemP = 256;
// NS = threads per query row (column slices of S): 4 -> 16 columns each (512 softmax threads), 2 -> 32 columns.
template <int NS>
__global__ void __launch_bounds__(128 * NS + 32, 1) extend_attend_tc5_kernel(const ExtendParams e) {
    constexpr int kTc5Softmax = 128 * NS;
    constexpr int W = 64 / NS;                               // S columns per thread
    constexpr int OW = 128 / NS;                             // O columns per thread
    extern __shared__ unsigned char tc5_dyn[];
    // the swizzled operand tiles need 1024-byte alignment
    Tc5Smem& sm = *reinterpret_cast<Tc5Smem*>(tc5_dyn + ((1024u - (smem_u32(tc5_dyn) & 1023u)) & 1023u));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = blockIdx.x, h = blockIdx.y, kv = h / e.group;
    const int lq = e.chunk_len;
    if (*(volatile int*)e.err != 0 || qt * 128 >= lq) return;
    const int count = min(*e.sel_count, e.n_sel);
    const int base_vis = count - lq;                         // query row r sees list entries j <= base_vis + r
    const int kmax = min(count - 1, base_vis + qt * 128 + 127);
    const int nblk = kmax / kTile + 1;
    bool dead = false;

    if (tid == 0) {
        mbar_init(smem_u32(&sm.qbar), 1);
        for (int s = 0; s < kKvStages; ++s) mbar_init(smem_u32(&sm.full[s]), 1);
        mbar_init(smem_u32(&sm.s_done[0]), 1);
        mbar_init(smem_u32(&sm.s_done[1]), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sm.o_done[i]), 1);
            mbar_init(smem_u32(&sm.p_ready[i]), kTc5Softmax / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t*)&sm.tmem_base;

    if (warp == kTc5Softmax / 32) {
        // ---------------- issuer ----------------
        if (lane == 0) {
            const unsigned char* qsrc = reinterpret_cast<const unsigned char*>(e.qc) + ((size_t)h * e.rows_q + (size_t)qt * 128) * 256;
            const unsigned char* ksrc = reinterpret_cast<const unsigned char*>(e.kc) + (size_t)kv * e.rows_k * 256;
            const unsigned char* vsrc = reinterpret_cast<const unsigned char*>(e.vc) + (size_t)kv * e.rows_k * 256;
            constexpr uint32_t kTileBytes = kTile * 256;     // one K or V tile image
            auto load_tile = [&](int b) {
                const int st = b % kKvStages;
                mbar_expect_tx(smem_u32(&sm.full[st]), 2 * kTileBytes);
                bulk_g2s(smem_u32(sm.k[st]), ksrc + (size_t)b * kTileBytes, kTileBytes, smem_u32(&sm.full[st]));
                bulk_g2s(smem_u32(sm.v[st]), vsrc + (size_t)b * kTileBytes, kTileBytes, smem_u32(&sm.full[st]));
            };
            // instruction descriptors: fp32 accumulate, bf16 A and B, M = 128; N = 64 with K-major B, N = 128 with MN-major B
            constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
            constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            auto issue_qk = [&](int b) {                     // S[b&1] = Q . K_b^T
                const int st = b % kKvStages;
                mbar_wait(smem_u32(&sm.full[st]), (uint32_t)((b / kKvStages) & 1), e.err, dead, 42, e.wait_cycles);
                tc_fence_after();
                const uint32_t qa = smem_u32(sm.q), ka = smem_u32(sm.k[st]);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off_q = (ks >> 2) * (128u * 128u) + (ks & 3) * 32u;
                    const uint32_t off_k = (ks >> 2) * (kTile * 128u) + (ks & 3) * 32u;
                    umma_bf16(tmem + 64u * (b & 1), umma_desc_sw128(qa + off_q, 16, 1024),
                              umma_desc_sw128(ka + off_k, 16, 1024), kIdescQK, ks > 0 ? 1u : 0u);
                }
                umma_commit(smem_u32(&sm.s_done[b & 1]));
            };
            mbar_expect_tx(smem_u32(&sm.qbar), 128 * 256);
            bulk_g2s(smem_u32(sm.q), qsrc, 128 * 256, smem_u32(&sm.qbar));
            for (int b = 0; b < kKvStages && b < nblk; ++b) load_tile(b);
            mbar_wait(smem_u32(&sm.qbar), 0, e.err, dead, 40, e.wait_cycles);
            issue_qk(0);
            for (int blk = 0; blk < nblk; ++blk) {
                if (blk + 1 < nblk) issue_qk(blk + 1);
                if (blk > 0 && blk - 1 + kKvStages < nblk) {
                    // P.V of the previous block is complete: its stage can take the tile four blocks ahead
                    mbar_wait(smem_u32(&sm.o_done[(blk - 1) & 1]), (uint32_t)(((blk - 1) >> 1) & 1), e.err, dead, 46, e.wait_cycles);
                    load_tile(blk - 1 + kKvStages);
                }
                mbar_wait(smem_u32(&sm.p_ready[blk & 1]), (uint32_t)((blk >> 1) & 1), e.err, dead, 47, e.wait_cycles);
                tc_fence_after();
                const uint32_t va = smem_u32(sm.v[blk % kKvStages]);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)               // 16 keys per step: 8 packed columns of P
                    umma_bf16_ts(tmem + kTmemO, tmem + kTmemP + 32u * (blk & 1) + 8u * ks,
                                 umma_desc_sw128(va + ks * 2048u, kTile * 128u, 1024), kIdescPV, (blk > 0 || ks > 0) ? 1u : 0u);
                umma_commit(smem_u32(&sm.o_done[blk & 1]));
            }
        }
    } else {
        // ---------------- softmax ----------------
        const int cq = warp >> 2, rq = warp & 3;             // column slice, row (lane) quarter
        const int r_in = rq * 32 + lane;                     // row inside the 128-row tile
        const uint32_t lane_base = (uint32_t)(rq * 32) << 16;
        const uint32_t t_s[2] = {tmem + lane_base + (uint32_t)(W * cq), tmem + lane_base + 64u + (uint32_t)(W * cq)};
        const uint32_t t_o = tmem + lane_base + kTmemO + (uint32_t)(OW * cq);
        const uint32_t t_p = tmem + lane_base + kTmemP + (uint32_t)(W / 2 * cq);
        const int row = qt * 128 + r_in;
        const int lim = base_vis + row;
        const float cap = e.logit_cap;
        const float mul = cap > 0.f ? 1.f : e.sm_scale * kLog2eX;     // x * mul is the logit in base-2 units
        float m_ref = 0.f, l_run = 0.f;

        for (int blk = 0; blk < nblk; ++blk) {
            mbar_wait(smem_u32(&sm.s_done[blk & 1]), (uint32_t)((blk >> 1) & 1), e.err, dead, 43, e.wait_cycles);
            tc_fence_after();
            float x[W];
            {
                uint32_t r0[W / 16][16];
#pragma unroll
                for (int j = 0; j < W / 16; ++j) tmem_ld16(t_s[blk & 1] + 16u * j, r0[j]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < W; ++c) x[c] = __uint_as_float(r0[c / 16][c % 16]);
            }
            // x keeps S in raw units unless the soft cap is on; the scale goes into the exponent's FMA
            float mx = -INFINITY;
            const int key0 = blk * kTile + W * cq;
            if (cap > 0.f) {
#pragma unroll
                for (int c = 0; c < W; ++c) x[c] = cap * tanhf(x[c] * e.sm_scale / cap) * kLog2eX;
            }
            if (blk * kTile + kTile - 1 > base_vis + qt * 128) {      // only blocks that reach the diagonal are masked
#pragma unroll
                for (int c = 0; c < W; ++c)
                    if (key0 + c > lim) x[c] = -INFINITY;
            }
#pragma unroll
            for (int c = 0; c < W; ++c) mx = fmaxf(mx, x[c]);
            mx *= mul;                                               // base-2 units (mul > 0)
            float* rm = &sm.rowmax[blk & 1][0][r_in];
            rm[cq * 128] = mx;
            named_bar_sync(1 + rq, 32 * NS);                 // the warps that share these rows
            mx = fmaxf(rm[0], rm[128]);
            if (NS == 4) mx = fmaxf(mx, fmaxf(rm[256], rm[384]));
            if (blk > 0) {
                const bool grow = mx > m_ref + 8.f;
                if (__any_sync(0xffffffffu, grow)) {
                    // O is rescaled in place: every P.V issued so far must be complete (they run in order)
                    mbar_wait(smem_u32(&sm.o_done[(blk - 1) & 1]), (uint32_t)(((blk - 1) >> 1) & 1), e.err, dead, 44, e.wait_cycles);
                    tc_fence_after();
                    const float corr = grow ? ex2_fast(m_ref - mx) : 1.f;
#pragma unroll
                    for (int j = 0; j < OW / 32; ++j) {
                        uint32_t r[32];
                        tmem_ld32(t_o + 32u * j, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * corr);
                        tmem_st32(t_o + 32u * j, r);
                    }
                    l_run *= corr;
                    if (grow) m_ref = mx;
                }
            } else {
                m_ref = mx == -INFINITY ? 0.f : mx;
            }
            float sum = 0.f;
            uint32_t w[W / 16][8];
#pragma unroll
            for (int u = 0; u < W / 2; ++u) {
                const float p0 = ex2_fast(fmaf(x[2 * u], mul, -m_ref)), p1 = ex2_fast(fmaf(x[2 * u + 1], mul, -m_ref));
                sum += p0 + p1;
                w[u / 8][u % 8] = pack_bf16(p0, p1);
            }
            if (blk >= 2) {                                  // P.V of block blk-2 has finished reading this P buffer
                mbar_wait(smem_u32(&sm.o_done[blk & 1]), (uint32_t)(((blk - 2) >> 1) & 1), e.err, dead, 48, e.wait_cycles);
                tc_fence_after();
            }
#pragma unroll
            for (int j = 0; j < W / 16; ++j) tmem_st8(t_p + 32u * (blk & 1) + 8u * j, w[j]);
            tmem_wait_st();
            l_run += sum;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.p_ready[blk & 1]));
        }
        // row sums: the four partial sums of a row share the reference maximum
        float* rs = &sm.rowmax[nblk & 1][0][r_in];
        rs[cq * 128] = l_run;
        named_bar_sync(1 + rq, 32 * NS);
        const float l_tot = NS == 4 ? (rs[0] + rs[128]) + (rs[256] + rs[384]) : rs[0] + rs[128];
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        mbar_wait(smem_u32(&sm.o_done[(nblk - 1) & 1]), (uint32_t)(((nblk - 1) >> 1) & 1), e.err, dead, 45, e.wait_cycles);
        tc_fence_after();
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(e.out) + (size_t)row * e.hq * 128 + (size_t)h * 128 + OW * cq;
#pragma unroll
        for (int j = 0; j < OW / 32; ++j) {
            uint32_t r[32];
            tmem_ld32(t_o + 32u * j, r);
            tmem_wait_ld();
            if (row < lq) {
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    uint4 w;
                    w.x = pack_bf16(__uint_as_float(r[c8 * 8 + 0]) * inv, __uint_as_float(r[c8 * 8 + 1]) * inv);
                    w.y = pack_bf16(__uint_as_float(r[c8 * 8 + 2]) * inv, __uint_as_float(r[c8 * 8 + 3]) * inv);
                    w.z = pack_bf16(__uint_as_float(r[c8 * 8 + 4]) * inv, __uint_as_float(r[c8 * 8 + 5]) * inv);
                    w.w = pack_bf16(__uint_as_float(r[c8 * 8 + 6]) * inv, __uint_as_float(r[c8 * 8 + 7]) * inv);
                    *reinterpret_cast<uint4*>(out + 32 * j + c8 * 8) = w;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// 4a''. key blocks of 128, loads issued by a warp of their own (the default)
// ------------------------------------------------------------------------------------------------
// What bounds the kernels above is neither the tensor pipe nor the softmax but the ONE thread that issues the
// asynchronous operations: measured on this part, every tcgen05.mma, tcgen05.commit, bulk copy and mbarrier
// wait costs that thread about 80 cycles, and a 64-key block needs two dozen of them (~1950 cycles per block
// against ~1060 cycles of softmax work and ~550 cycles of tensor-pipe time).  Two softmax teams on alternating
// blocks did not help for that reason.  This form halves the operations per key: blocks of 128 keys (Q.K^T as
// eight M128 x N128 x K16 MMAs instead of sixteen N64 ones, one commit and one tile request per 128 keys), and
// the tile requests and the waits that guard them moved to a second single-thread warp.
//   S[b&1]  128 x 128 fp32, TMEM columns 128 (b&1) ..
//   O       128 x 128 fp32, TMEM columns 256 .. 383
//   P[b&1]  128 x 128 packed bf16 = 64 columns, TMEM columns 384 + 64 (b&1) ..
// TWO issuing threads (different warps): one issues every Q.K^T as soon as the S buffer has been read (two blocks
// ahead of the softmax), the other every P.V as soon as P is written; they touch disjoint tensor memory (S / O, P),
// and every dependency between them and the softmax goes through an mbarrier (S written -> s_done, S read and P
// written -> p_ready, P read -> o_done).
// 512 softmax threads: thread (column quarter c = warp / 4, lane quarter w = warp % 4, lane l) owns query row
// 32 w + l and columns [32 c, 32 c + 32) of S and of O.  K tiles (32 KB) have two stages, freed as soon as their
// Q.K^T has run; V tiles three, freed after their P.V.
constexpr int kWide = 128;                                   // keys per block
constexpr int kWideKStages = 2, kWideVStages = 3;
struct Tc5WideSmem {
    unsigned char q[128 * 256];                  // 2 halves x [128 rows][128 B]
    unsigned char k[kWideKStages][kWide * 256];  // 2 halves x [128 keys][128 B]
    unsigned char v[kWideVStages][kWide * 256];
    float rowmax[2][4][128];                     // [block parity][column quarter][row]: row maxima; row sums at the end
    uint64_t qbar, full_k[kWideKStages], full_v[kWideVStages], s_done[4], o_done[4], p_ready[2];
    uint32_t tmem_base;
};
static_assert(sizeof(Tc5WideSmem) + 1024 <= 232448, "the kernel's shared memory must fit one CTA's maximum");

__global__ void __launch_bounds__(608, 1) extend_attend_tc5_wide_kernel(const ExtendParams e) {
    constexpr int W = 32;                                    // S columns per thread
    constexpr int OW = 32;                                   // O columns per thread
    constexpr uint32_t kWideO = 256, kWideP = 384;            // TMEM columns of O and of the two P buffers (64 each)
    extern __shared__ unsigned char tc5_dyn[];
    Tc5WideSmem& sm = *reinterpret_cast<Tc5WideSmem*>(tc5_dyn + ((1024u - (smem_u32(tc5_dyn) & 1023u)) & 1023u));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = blockIdx.x, h = blockIdx.y, kv = h / e.group;
    const int lq = e.chunk_len;
    if (qt * 128 >= lq) return;
    bool dead = false;

    if (tid == 0) {
        mbar_init(smem_u32(&sm.qbar), 1);
        for (int s = 0; s < kWideKStages; ++s) mbar_init(smem_u32(&sm.full_k[s]), 1);
        for (int s = 0; s < kWideVStages; ++s) mbar_init(smem_u32(&sm.full_v[s]), 1);
        for (int s = 0; s < 4; ++s) {
            mbar_init(smem_u32(&sm.s_done[s]), 1);
            mbar_init(smem_u32(&sm.o_done[s]), 1);
        }
        mbar_init(smem_u32(&sm.p_ready[0]), 16);             // the sixteen softmax warps
        mbar_init(smem_u32(&sm.p_ready[1]), 16);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t*)&sm.tmem_base;
    constexpr uint32_t kTileBytes = kWide * 256;             // one K or V tile image
    // Launched with programmatic stream serialization: everything above touched only this CTA's shared and tensor
    // memory and ran while the gather kernel was finishing; nothing global is read before this wait.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const bool skip = *(volatile int*)e.err != 0;            // a handle in error: no work, but the tensor memory is freed
    const int count = min(*e.sel_count, e.n_sel);
    const int base_vis = count - lq;                         // query row r sees list entries j <= base_vis + r
    const int kmax = min(count - 1, base_vis + qt * 128 + 127);
    const int nblk = kmax / kWide + 1;
    const bool timed_cta = e.stamps != nullptr && qt == 0 && h == 0;      // cycle counts under TS_CFG_PHASE_STAMPS

    if (skip) {
    } else if (warp == 18) {
        // ---------------- loader: one thread requests every tile ----------------
        if (lane == 0) {
            const unsigned char* qsrc = reinterpret_cast<const unsigned char*>(e.qc) + ((size_t)h * e.rows_q + (size_t)qt * 128) * 256;
            const unsigned char* ksrc = reinterpret_cast<const unsigned char*>(e.kc) + (size_t)kv * e.rows_k * 256;
            const unsigned char* vsrc = reinterpret_cast<const unsigned char*>(e.vc) + (size_t)kv * e.rows_k * 256;
            mbar_expect_tx(smem_u32(&sm.qbar), 128 * 256);
            bulk_g2s(smem_u32(sm.q), qsrc, 128 * 256, smem_u32(&sm.qbar));
            for (int b = 0; b < nblk; ++b) {
                if (b >= kWideKStages) {                     // the stage's previous tile: its Q.K^T has run
                    const int pb = b - kWideKStages;
                    mbar_wait(smem_u32(&sm.s_done[pb & 3]), (uint32_t)((pb >> 2) & 1), e.err, dead, 46, e.wait_cycles);
                }
                mbar_expect_tx(smem_u32(&sm.full_k[b % kWideKStages]), kTileBytes);
                bulk_g2s(smem_u32(sm.k[b % kWideKStages]), ksrc + (size_t)b * kTileBytes, kTileBytes, smem_u32(&sm.full_k[b % kWideKStages]));
                if (b >= kWideVStages) {                     // the stage's previous tile: its P.V has run
                    const int pb = b - kWideVStages;
                    mbar_wait(smem_u32(&sm.o_done[pb & 3]), (uint32_t)((pb >> 2) & 1), e.err, dead, 49, e.wait_cycles);
                }
                mbar_expect_tx(smem_u32(&sm.full_v[b % kWideVStages]), kTileBytes);
                bulk_g2s(smem_u32(sm.v[b % kWideVStages]), vsrc + (size_t)b * kTileBytes, kTileBytes, smem_u32(&sm.full_v[b % kWideVStages]));
            }
        }
    } else if (warp == 16) {
        // ---------------- first issuing thread: every Q.K^T ----------------
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, bf16 A and B, M = 128, N = 128, B K-major
            constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            long long w_k = 0, w_s = 0, c0 = 0;
            const long long t_begin = clock64();
            mbar_wait(smem_u32(&sm.qbar), 0, e.err, dead, 40, e.wait_cycles);
            for (int b = 0; b < nblk; ++b) {
                if (timed_cta) c0 = clock64();
                if (b >= 2) {                                // the S buffer's previous block has been read by the softmax
                    const int pb = b - 2;
                    mbar_wait(smem_u32(&sm.p_ready[pb & 1]), (uint32_t)((pb >> 1) & 1), e.err, dead, 47, e.wait_cycles);
                }
                if (timed_cta) { const long long c = clock64(); w_s += c - c0; c0 = c; }
                const int st = b % kWideKStages;
                mbar_wait(smem_u32(&sm.full_k[st]), (uint32_t)((b / kWideKStages) & 1), e.err, dead, 42, e.wait_cycles);
                tc_fence_after();
                const uint32_t qa = smem_u32(sm.q), ka = smem_u32(sm.k[st]);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off_q = (ks >> 2) * (128u * 128u) + (ks & 3) * 32u;
                    const uint32_t off_k = (ks >> 2) * (kWide * 128u) + (ks & 3) * 32u;
                    umma_bf16(tmem + 128u * (b & 1), umma_desc_sw128(qa + off_q, 16, 1024),
                              umma_desc_sw128(ka + off_k, 16, 1024), kIdescQK, ks > 0 ? 1u : 0u);
                }
                umma_commit(smem_u32(&sm.s_done[b & 3]));
                if (timed_cta) { const long long c = clock64(); w_k += c - c0; c0 = c; }
            }
            if (timed_cta) {
                e.stamps[64] = (unsigned long long)(clock64() - t_begin);     // its whole loop
                e.stamps[65] = (unsigned long long)w_k;                        // wait for the K tile, 8 MMAs, commit
                e.stamps[66] = (unsigned long long)w_s;                        // wait for the S buffer
                e.stamps[69] = (unsigned long long)nblk;
            }
        }
    } else if (warp == 17) {
        // ---------------- second issuing thread: every P.V ----------------
        if (lane == 0) {
            // fp32 accumulate, bf16 A (tensor memory) and B (MN-major), M = 128, N = 128
            constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            long long w_p = 0, w_v = 0, w_i = 0, c0 = 0;
            for (int blk = 0; blk < nblk; ++blk) {
                if (timed_cta) c0 = clock64();
                mbar_wait(smem_u32(&sm.p_ready[blk & 1]), (uint32_t)((blk >> 1) & 1), e.err, dead, 47, e.wait_cycles);
                if (timed_cta) { const long long c = clock64(); w_p += c - c0; c0 = c; }
                mbar_wait(smem_u32(&sm.full_v[blk % kWideVStages]), (uint32_t)((blk / kWideVStages) & 1), e.err, dead, 41, e.wait_cycles);
                if (timed_cta) { const long long c = clock64(); w_v += c - c0; c0 = c; }
                tc_fence_after();
                const uint32_t va = smem_u32(sm.v[blk % kWideVStages]);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)               // 16 keys per step: 8 packed columns of P
                    umma_bf16_ts(tmem + kWideO, tmem + kWideP + 64u * (blk & 1) + 8u * ks,
                                 umma_desc_sw128(va + ks * 2048u, kWide * 128u, 1024), kIdescPV, (blk > 0 || ks > 0) ? 1u : 0u);
                umma_commit(smem_u32(&sm.o_done[blk & 3]));
                if (timed_cta) { const long long c = clock64(); w_i += c - c0; c0 = c; }
            }
            if (timed_cta) {
                e.stamps[67] = (unsigned long long)w_p;                        // wait for P
                e.stamps[68] = (unsigned long long)w_v;                        // wait for the V tile
                e.stamps[70] = (unsigned long long)w_i;                        // 8 MMAs, commit
            }
        }
    } else {
        // ---------------- softmax ----------------
        const int cq = warp >> 2, rq = warp & 3;             // column quarter, row (lane) quarter
        const int r_in = rq * 32 + lane;                     // row inside the 128-row tile
        const uint32_t lane_base = (uint32_t)(rq * 32) << 16;
        const uint32_t t_o = tmem + lane_base + kWideO + (uint32_t)(OW * cq);
        const int row = qt * 128 + r_in;
        const int lim = base_vis + row;
        const float cap = e.logit_cap;
        const float mul = cap > 0.f ? 1.f : e.sm_scale * kLog2eX;     // x * mul is the logit in base-2 units
        float m_ref = 0.f, l_run = 0.f;
        const bool timed = timed_cta && warp == 0 && lane == 0;
        long long c_s = 0, c_ld = 0, c_bar = 0, c_exp = 0, c_st = 0, c0 = 0;
        const long long t_begin = clock64();

        for (int blk = 0; blk < nblk; ++blk) {
            const uint32_t t_s = tmem + lane_base + 128u * (blk & 1) + (uint32_t)(W * cq);
            const uint32_t t_p = tmem + lane_base + kWideP + 64u * (blk & 1) + (uint32_t)(W / 2 * cq);
            if (timed) c0 = clock64();
            mbar_wait(smem_u32(&sm.s_done[blk & 3]), (uint32_t)((blk >> 2) & 1), e.err, dead, 43, e.wait_cycles);
            tc_fence_after();
            if (timed) { const long long c = clock64(); c_s += c - c0; c0 = c; }
            float x[W];
            {
                uint32_t r0[W / 16][16];
#pragma unroll
                for (int j = 0; j < W / 16; ++j) tmem_ld16(t_s + 16u * j, r0[j]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < W; ++c) x[c] = __uint_as_float(r0[c / 16][c % 16]);
            }
            if (timed) { const long long c = clock64(); c_ld += c - c0; c0 = c; }
            // x keeps S in raw units unless the soft cap is on; the scale goes into the exponent's FMA
            float mx = -INFINITY;
            const int key0 = blk * kWide + W * cq;
            if (cap > 0.f) {
#pragma unroll
                for (int c = 0; c < W; ++c) x[c] = cap * tanhf(x[c] * e.sm_scale / cap) * kLog2eX;
            }
            if (blk * kWide + kWide - 1 > base_vis + qt * 128) {      // only blocks that reach the diagonal are masked
#pragma unroll
                for (int c = 0; c < W; ++c)
                    if (key0 + c > lim) x[c] = -INFINITY;
            }
#pragma unroll
            for (int c = 0; c < W; ++c) mx = fmaxf(mx, x[c]);
            mx *= mul;                                               // base-2 units (mul > 0)
            float* rm = &sm.rowmax[blk & 1][0][r_in];
            rm[cq * 128] = mx;
            named_bar_sync(1 + rq, 128);                     // the four warps that share these rows
            mx = fmaxf(fmaxf(rm[0], rm[128]), fmaxf(rm[256], rm[384]));
            if (timed) { const long long c = clock64(); c_bar += c - c0; c0 = c; }
            if (blk > 0) {
                const bool grow = mx > m_ref + 8.f;
                if (__any_sync(0xffffffffu, grow)) {
                    // O is rescaled in place: every P.V issued so far must be complete (they run in order)
                    mbar_wait(smem_u32(&sm.o_done[(blk - 1) & 3]), (uint32_t)(((blk - 1) >> 2) & 1), e.err, dead, 44, e.wait_cycles);
                    tc_fence_after();
                    const float corr = grow ? ex2_fast(m_ref - mx) : 1.f;
#pragma unroll 1
                    for (int j = 0; j < OW / 16; ++j) {
                        uint32_t r[16];
                        tmem_ld16(t_o + 16u * j, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 16; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * corr);
                        tmem_st16(t_o + 16u * j, r);
                    }
                    l_run *= corr;
                    if (grow) m_ref = mx;
                }
            } else {
                m_ref = mx == -INFINITY ? 0.f : mx;
            }
            float sum = 0.f;
            uint32_t w[W / 16][8];
#pragma unroll
            for (int c = 0; c < W / 2; ++c) {
                const float p0 = ex2_fast(fmaf(x[2 * c], mul, -m_ref)), p1 = ex2_fast(fmaf(x[2 * c + 1], mul, -m_ref));
                sum += p0 + p1;
                w[c / 8][c % 8] = pack_bf16(p0, p1);
            }
            if (timed) { const long long c = clock64(); c_exp += c - c0; c0 = c; }
            if (blk >= 2) {                                  // P.V of block blk-2 has finished reading this P buffer
                mbar_wait(smem_u32(&sm.o_done[(blk - 2) & 3]), (uint32_t)(((blk - 2) >> 2) & 1), e.err, dead, 48, e.wait_cycles);
                tc_fence_after();
            }
#pragma unroll
            for (int j = 0; j < W / 16; ++j) tmem_st8(t_p + 8u * j, w[j]);
            tmem_wait_st();
            l_run += sum;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.p_ready[blk & 1]));
            if (timed) { const long long c = clock64(); c_st += c - c0; c0 = c; }
        }
        if (timed) {
            unsigned long long* o = e.stamps + 72;
            o[0] = (unsigned long long)(clock64() - t_begin);   // the softmax loop
            o[1] = (unsigned long long)c_s;                      // wait for S
            o[2] = (unsigned long long)c_ld;                     // tcgen05.ld + wait
            o[3] = (unsigned long long)c_bar;                    // mask, maximum, exchange with the other column quarters
            o[4] = (unsigned long long)c_exp;                    // (rescale,) exponentials, pack
            o[5] = (unsigned long long)c_st;                     // tcgen05.st + wait, arrive
            o[6] = (unsigned long long)nblk;
        }
        // row sums: the four partial sums of a row share the reference maximum
        float* rs = &sm.rowmax[nblk & 1][0][r_in];
        rs[cq * 128] = l_run;
        named_bar_sync(1 + rq, 128);
        const float l_tot = (rs[0] + rs[128]) + (rs[256] + rs[384]);
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        mbar_wait(smem_u32(&sm.o_done[(nblk - 1) & 3]), (uint32_t)(((nblk - 1) >> 2) & 1), e.err, dead, 45, e.wait_cycles);
        tc_fence_after();
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(e.out) + (size_t)row * e.hq * 128 + (size_t)h * 128 + OW * cq;
#pragma unroll 1
        for (int j = 0; j < OW / 16; ++j) {
            uint32_t r[16];
            tmem_ld16(t_o + 16u * j, r);
            tmem_wait_ld();
            if (row < lq) {
#pragma unroll
                for (int c8 = 0; c8 < 2; ++c8) {
                    uint4 w;
                    w.x = pack_bf16(__uint_as_float(r[c8 * 8 + 0]) * inv, __uint_as_float(r[c8 * 8 + 1]) * inv);
                    w.y = pack_bf16(__uint_as_float(r[c8 * 8 + 2]) * inv, __uint_as_float(r[c8 * 8 + 3]) * inv);
                    w.z = pack_bf16(__uint_as_float(r[c8 * 8 + 4]) * inv, __uint_as_float(r[c8 * 8 + 5]) * inv);
                    w.w = pack_bf16(__uint_as_float(r[c8 * 8 + 6]) * inv, __uint_as_float(r[c8 * 8 + 7]) * inv);
                    *reinterpret_cast<uint4*>(out + 16 * j + c8 * 8) = w;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
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
    const int groups = e.hq * (e.d / 2) / 8;
    const int fp_blocks = (groups + 1) / 2;
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
    const int per_block = kExtThreads / (half / 8);
    const bool tc5 = tc && !(l.flags & TS_CFG_EXTEND_MMA_SYNC);
    const bool wide = tc5 && !(l.flags & (TS_CFG_EXTEND_FOUR_PER_ROW | TS_CFG_EXTEND_NARROW_BLOCKS));
    const int layout = tc5 ? kLayoutImage : tc ? kLayoutXor16 : kLayoutPlain;
    const int kv_tile = wide ? kWide : kTile;                // keys per K / V tile image
    stage_begin(l, kStageExtendGather);
    if (l.dtype == TS_DTYPE_BF16)
        extend_gather_kernel<__nv_bfloat16><<<(items + per_block - 1) / per_block, kExtThreads, 0, l.stream>>>(e, layout, kv_tile);
    else
        extend_gather_kernel<float><<<(items + per_block - 1) / per_block, kExtThreads, 0, l.stream>>>(e, layout, kv_tile);
    stage_end(l);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    stage_begin(l, kStageExtendAttend);
    if (tc5) {
        static SmemConfig configured5 = {};
        const size_t smem5 = sizeof(Tc5Smem) + 1024;
        if (wide) {
            static SmemConfig configured_wide = {};
            const size_t smem_wide = sizeof(Tc5WideSmem) + 1024;
            err = ensure_dynamic_smem(extend_attend_tc5_wide_kernel, smem_wide, configured_wide);
            if (err != cudaSuccess) return err;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(e.rows_q / 128, e.hq);
            cfg.blockDim = dim3(608);
            cfg.dynamicSmemBytes = smem_wide;
            cfg.stream = l.stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            err = cudaLaunchKernelEx(&cfg, extend_attend_tc5_wide_kernel, e);
            if (err != cudaSuccess) return err;
        } else if (!(l.flags & TS_CFG_EXTEND_FOUR_PER_ROW)) {
            static SmemConfig configured2 = {};
            err = ensure_dynamic_smem(extend_attend_tc5_kernel<2>, smem5, configured2);
            if (err != cudaSuccess) return err;
            extend_attend_tc5_kernel<2><<<dim3(e.rows_q / 128, e.hq), 128 * 2 + 32, smem5, l.stream>>>(e);
        } else {
            err = ensure_dynamic_smem(extend_attend_tc5_kernel<4>, smem5, configured5);
            if (err != cudaSuccess) return err;
            extend_attend_tc5_kernel<4><<<dim3(e.rows_q / 128, e.hq), 128 * 4 + 32, smem5, l.stream>>>(e);
        }
    } else if (tc) {
        static SmemConfig configured = {};
        err = ensure_dynamic_smem(extend_attend_tc_kernel, sizeof(ExtSmem), configured);
        if (err != cudaSuccess) return err;
        extend_attend_tc_kernel<<<dim3(e.rows_q / kQTile, e.hq), 128, sizeof(ExtSmem), l.stream>>>(e);
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
