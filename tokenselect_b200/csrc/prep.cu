// Rotation tables and the stand-alone prepare kernel of the tensor-parallel form (the cosine terms
// it publishes are summed over ranks before the decision).  See prep.cuh.
#include "prep.cuh"

namespace ts {

// cos/sin tables: row r of attn_cs holds position r with frequencies divided by rope_scale
// (the decode wrapper's convention, :820-822); score_cs holds position n_local*rope_scale (:93).
__global__ void rope_table_kernel(float2* score_cs, float2* attn_cs, int d, int n_rows, double base,
                                  double rope_scale, int n_local) {
    int half = d / 2;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (n_rows + 1) * half) return;
    int row = idx / half, i = idx % half;
    // fp32 inverse frequency, rounded once from a double evaluation
    float inv = (float)(1.0 / pow(base, (double)(2 * i) / (double)d));
    if (row == n_rows) {
        float ang = __fmul_rn((float)((double)n_local * rope_scale), inv);
        score_cs[i] = make_float2(cosf(ang), sinf(ang));
    } else {
        float ang = __fmul_rn((float)row, (float)(inv / (float)rope_scale));
        attn_cs[(size_t)row * half + i] = make_float2(cosf(ang), sinf(ang));
    }
}

cudaError_t launch_rope_tables(float2* score_cs, float2* attn_cs, int d, int n_rows, double base,
                               double rope_scale, int n_local, cudaStream_t stream) {
    int total = (n_rows + 1) * (d / 2);
    rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(score_cs, attn_cs, d, n_rows, base,
                                                               rope_scale, n_local);
    return cudaGetLastError();
}

__global__ void lane_order_kernel(const float2* src, float2* dst, int half, int n_rows) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * half) return;
    const int row = idx / half, i = idx - row * half;
    dst[(size_t)row * half + lane_order_slot(i, half / 8)] = src[idx];
}

cudaError_t launch_lane_order_table(const float2* attn_cs, float2* attn_cs_lane, int d, int n_rows, cudaStream_t stream) {
    const int total = n_rows * (d / 2);
    lane_order_kernel<<<(total + 255) / 256, 256, 0, stream>>>(attn_cs, attn_cs_lane, d / 2, n_rows);
    return cudaGetLastError();
}

// Tile order for the tensor-core attention kernel (head_dim 128): positions in tiles of eight; inside a
// tile the (cos, sin) of frequency i = 16s + 8u + 2t + w of position g sits in float4 ((s*2+u)*8 + g)*4 + t,
// halves w = 0, 1 -- the order in which a warp's lanes (g = lane/4, t = lane%4) need them, so that one
// 16-byte load per lane is conflict-free.
__global__ void tile_order_kernel(const float2* src, float2* dst, int n_rows, int n_tiles) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tiles * 8 * 64) return;
    const int pos = idx / 64, i = idx - pos * 64;
    const int tile = pos >> 3, g = pos & 7;
    const int s = i >> 4, u = (i >> 3) & 1, t = (i >> 1) & 3, w = i & 1;
    const float2 v = pos < n_rows ? src[(size_t)pos * 64 + i] : make_float2(1.f, 0.f);
    dst[((size_t)tile * 256 + ((s * 2 + u) * 8 + g) * 4 + t) * 2 + w] = v;
}

cudaError_t launch_tile_order_table(const float2* attn_cs, float4* attn_cs_tile, int n_rows, int n_tiles, cudaStream_t stream) {
    const int total = n_tiles * 8 * 64;
    tile_order_kernel<<<(total + 255) / 256, 256, 0, stream>>>(attn_cs, reinterpret_cast<float2*>(attn_cs_tile), n_rows, n_tiles);
    return cudaGetLastError();
}

// Rotation frequency i of the attention positions, recovered from the table's row of position 1
// (angle = 1 * frequency, far below pi): the in-kernel attention rotates at positions it only learns at run
// time and evaluates cos/sin of position * frequency itself.
__global__ void inv_freq_kernel(const float2* attn_cs, float* inv_freq, int half) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < half) inv_freq[i] = atan2f(attn_cs[half + i].y, attn_cs[half + i].x);
}
cudaError_t launch_inv_freq_table(const float2* attn_cs, float* inv_freq, int d, cudaStream_t stream) {
    inv_freq_kernel<<<1, 128, 0, stream>>>(attn_cs, inv_freq, d / 2);
    return cudaGetLastError();
}

// grid = batch, block = 256.
template <typename T>
__global__ void __launch_bounds__(256) prep_kernel(const LayerParams p) {
    __shared__ PrepShared ps;
    if (*(volatile int*)p.err != 0) return;
    prepare_request<T, false>(p, blockIdx.x, ps, whole_cta());
}

cudaError_t launch_prep(const LayerParams& p, const Launch& l) {
    dim3 grid(p.batch), block(256);
    stage_begin(l, kStagePrep);
    if (l.dtype == TS_DTYPE_BF16) prep_kernel<__nv_bfloat16><<<grid, block, 0, l.stream>>>(p);
    else prep_kernel<float><<<grid, block, 0, l.stream>>>(p);
    stage_end(l);
    return cudaGetLastError();
}

}  // namespace ts
