// ts_attend_rows_static: sparse paged decode attention over a caller-supplied list of pool rows, for
// callers that must not allocate.
//
// Who that is: code that runs where device allocation is forbidden or impossible -- a host callback or a
// latency-critical serving loop that is not allowed to touch the allocator (cudaMalloc can synchronise the
// device), or a process whose device memory was handed out in full at start-up (to the KV pool, say) and
// whose owner gives out no more.  Such a caller cannot use ts_create(), which makes one cudaMalloc for its
// workspace.  This entry point needs no handle: the split kernel's partial results go
// to a fixed array that is part of the library image, the caller passes only inputs and the output.
//
// The array is shared by every call in the process and keeps whatever the last call left in it.  Nothing
// in it has to start at zero (every partial that the merge reads is written by the split of the same
// call).  Two calls whose kernels overlap on the GPU (different streams, no ordering) race on it.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress).  That first call
// should be made before any stream capture begins.
//
// Same arithmetic as csrc/attend.cu (query rotated at position count-1, j-th listed key at position j,
// rotate-half pairing, logits * sm_scale, optional soft cap, fp32 softmax, KV head = h / group), except
// that cos/sin are evaluated in the kernel instead of being read from the handle's tables.
#include <math.h>

#include "common.cuh"

namespace ts {

constexpr size_t kStaticScratchBytes = 4u << 20;       // 4 MiB, held by every GPU that loads the library
constexpr int kStaticChunk = 32;                        // listed rows per split CTA
constexpr int kStaticMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticParams {
    const void* q;
    const void* k_pool;
    const void* v_pool;
    const int* rows;
    void* out;
    float* scratch;                 // [chunks][hq][d + 2]: o[d], max (base-2 units), sum
    long long pool_rows;
    int hq, hkv, d, count, chunks;
    float sm_scale, logit_cap;
    double log2_base, rope_scale;
    int* status;                    // optional device int: set to TS_ERR_BAD_SLOT on a row outside the pool
};

// grid (chunks, hkv), block 128.  Warp w takes rows w, w+4, ... of the chunk; lane l holds elements
// [P*l, P*l+P) of both halves of a row (P = d/64), i.e. both members of each rotation pair.
template <typename T, int P>
__global__ void __launch_bounds__(128) static_split_kernel(const StaticParams p) {
    constexpr int D = 64 * P, HALF = 32 * P;
    __shared__ float sm_o[4][8][D];
    __shared__ float2 sm_ml[4][8];
    const int chunk = blockIdx.x, kv = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.hq / p.hkv;
    const int base = chunk * kStaticChunk;
    const int cnt = min(kStaticChunk, p.count - base);
    const T* kpool = reinterpret_cast<const T*>(p.k_pool);
    const T* vpool = reinterpret_cast<const T*>(p.v_pool);
    const T* q = reinterpret_cast<const T*>(p.q);

    float inv_freq[P];
#pragma unroll
    for (int e = 0; e < P; ++e)
        inv_freq[e] = (float)(exp2(-p.log2_base * (double)(2 * (P * lane + e)) / (double)D) / p.rope_scale);

    for (int g = 0; g < G; ++g) {
        const int h = kv * G + g;
        float q1[P], q2[P];
#pragma unroll
        for (int e = 0; e < P; ++e) {
            float s, c;
            sincosf(__fmul_rn((float)(p.count - 1), inv_freq[e]), &s, &c);
            const float x1 = to_f32<T>(q[h * D + P * lane + e]), x2 = to_f32<T>(q[h * D + HALF + P * lane + e]);
            q1[e] = x1 * c - x2 * s;
            q2[e] = x2 * c + x1 * s;
        }
        float m = -INFINITY, l = 0.f, o1[P], o2[P];
#pragma unroll
        for (int e = 0; e < P; ++e) { o1[e] = 0.f; o2[e] = 0.f; }
        for (int j = warp; j < cnt; j += 4) {
            int row = __ldg(p.rows + base + j);
            if ((unsigned long long)(long long)row >= (unsigned long long)p.pool_rows) {
                if (p.status != nullptr && lane == 0) atomicCAS(p.status, 0, TS_ERR_BAD_SLOT);
                row = 0;
            }
            const T* kr = kpool + ((size_t)row * p.hkv + kv) * D;
            const T* vr = vpool + ((size_t)row * p.hkv + kv) * D;
            float acc = 0.f, v1[P], v2[P];
#pragma unroll
            for (int e = 0; e < P; ++e) {
                float s, c;
                sincosf(__fmul_rn((float)(base + j), inv_freq[e]), &s, &c);
                const float x1 = to_f32<T>(kr[P * lane + e]), x2 = to_f32<T>(kr[HALF + P * lane + e]);
                acc += q1[e] * (x1 * c - x2 * s) + q2[e] * (x2 * c + x1 * s);
                v1[e] = to_f32<T>(vr[P * lane + e]);
                v2[e] = to_f32<T>(vr[HALF + P * lane + e]);
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            float x = acc * p.sm_scale;
            if (p.logit_cap > 0.f) x = p.logit_cap * tanhf(x / p.logit_cap);
            x *= 1.4426950408889634f;
            const float mn = fmaxf(m, x);
            const float sc = exp2f(m - mn), pe = exp2f(x - mn);
            l = l * sc + pe;
            m = mn;
#pragma unroll
            for (int e = 0; e < P; ++e) { o1[e] = o1[e] * sc + pe * v1[e]; o2[e] = o2[e] * sc + pe * v2[e]; }
        }
#pragma unroll
        for (int e = 0; e < P; ++e) { sm_o[warp][g][P * lane + e] = o1[e]; sm_o[warp][g][HALF + P * lane + e] = o2[e]; }
        if (lane == 0) sm_ml[warp][g] = make_float2(m, l);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += 128) {
        const int g = idx / D, e = idx - g * D;
        float mm = -INFINITY;
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_ml[w][g].x);
        float acc = 0.f, ll = 0.f;
        for (int w = 0; w < 4; ++w) {
            const float2 ml = sm_ml[w][g];
            const float wgt = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - mm);
            acc += sm_o[w][g][e] * wgt;
            ll += ml.y * wgt;
        }
        float* dst = p.scratch + ((size_t)chunk * p.hq + kv * G + g) * (D + 2);
        dst[e] = acc;
        if (e == 0) { dst[D] = mm; dst[D + 1] = ll; }
    }
}

// grid hq, block d.
template <typename T>
__global__ void static_merge_kernel(const StaticParams p) {
    const int h = blockIdx.x, e = threadIdx.x, D = p.d;
    float mm = -INFINITY;
    for (int c = 0; c < p.chunks; ++c) mm = fmaxf(mm, p.scratch[((size_t)c * p.hq + h) * (D + 2) + D]);
    float acc = 0.f, ll = 0.f;
    for (int c = 0; c < p.chunks; ++c) {
        const float* src = p.scratch + ((size_t)c * p.hq + h) * (D + 2);
        const float w = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - mm);
        acc += src[e] * w;
        ll += src[D + 1] * w;
    }
    reinterpret_cast<T*>(p.out)[(size_t)h * D + e] = from_f32<T>(acc / ll);
}

}  // namespace ts

extern "C" int ts_attend_rows_static(const ts_attend_static_args* a) {
    using namespace ts;
    if (!a || a->struct_size != sizeof(ts_attend_static_args)) return TS_ERR_INVALID_ARG;
    if (!a->q || !a->k_pool || !a->v_pool || !a->rows || !a->out) return TS_ERR_INVALID_ARG;
    if (a->hq < 1 || a->hkv < 1 || a->hq % a->hkv != 0 || a->count < 1 || a->pool_rows < 1) return TS_ERR_INVALID_ARG;
    if (a->dtype != TS_DTYPE_BF16 && a->dtype != TS_DTYPE_F32) return TS_ERR_UNSUPPORTED;
    if (a->head_dim != 64 && a->head_dim != 128) return TS_ERR_UNSUPPORTED;
    if (a->hq / a->hkv > 8) return TS_ERR_UNSUPPORTED;
    if (!(a->rope_base > 0.0) || !(a->rope_scale > 0.0)) return TS_ERR_INVALID_ARG;
    const int chunks = (a->count + kStaticChunk - 1) / kStaticChunk;
    // the fixed array bounds the list length: chunks * hq * (head_dim + 2) floats must fit in 4 MiB
    if ((size_t)chunks * a->hq * (a->head_dim + 2) * sizeof(float) > kStaticScratchBytes) return TS_ERR_CAPACITY;

    // One-time set-up per device, with that device current: the array's name is only a host-side handle
    // here; kernels need its device address.
    static float* scratch_of_device[kStaticMaxDevices] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return TS_ERR_CUDA;
    if (scratch_of_device[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return TS_ERR_CUDA;
        scratch_of_device[dev] = static_cast<float*>(ptr);
    }

    StaticParams p;
    p.q = a->q; p.k_pool = a->k_pool; p.v_pool = a->v_pool; p.rows = a->rows; p.out = a->out;
    p.scratch = scratch_of_device[dev];
    p.pool_rows = a->pool_rows;
    p.hq = a->hq; p.hkv = a->hkv; p.d = a->head_dim; p.count = a->count; p.chunks = chunks;
    p.sm_scale = a->sm_scale; p.logit_cap = a->logit_cap;
    p.log2_base = log2(a->rope_base); p.rope_scale = a->rope_scale;
    p.status = a->status;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(a->stream);
    dim3 grid(chunks, a->hkv);
    if (a->dtype == TS_DTYPE_BF16) {
        if (a->head_dim == 128) static_split_kernel<__nv_bfloat16, 2><<<grid, 128, 0, s>>>(p);
        else static_split_kernel<__nv_bfloat16, 1><<<grid, 128, 0, s>>>(p);
        static_merge_kernel<__nv_bfloat16><<<a->hq, a->head_dim, 0, s>>>(p);
    } else {
        if (a->head_dim == 128) static_split_kernel<float, 2><<<grid, 128, 0, s>>>(p);
        else static_split_kernel<float, 1><<<grid, 128, 0, s>>>(p);
        static_merge_kernel<float><<<a->hq, a->head_dim, 0, s>>>(p);
    }
    return cudaGetLastError() == cudaSuccess ? TS_OK : TS_ERR_CUDA;
}
