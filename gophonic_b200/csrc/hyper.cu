// Hyper-connections: the residual is S streams x_0 .. x_(S-1), each [rows, width] float32.  Around a
// sublayer two row-wise steps touch them,
//
//     write:  x_t <- sum_s mix[s, t] x_s + mult * out[t] * y      (all t from the old streams)
//     read:   u = sum_s in[s] x_s;   x_out = u / sqrt(mean(u^2) + eps) * w
//
// and between two sublayers the write of one is followed by the read of the next on the same rows.
// One kernel does either or both in one pass over a row: a thread takes a column's S values and the
// sublayer's output, forms the new values, stores them, and keeps the column's u in shared memory for
// the norm that follows the row's sum of squares.  Everything is float32 but the normed output, which is
// written in the activation dtype.  With a row index (the final norm of the wanted rows) the new values
// are formed for the picked rows only and nothing is written back.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace {

constexpr int HC_MAX_THREADS = 1024;

template <typename TO, int S>
__global__ void __launch_bounds__(HC_MAX_THREADS) hyper_mix_norm_kernel(HyperParams p) {
    extern __shared__ float u_s[];          // the row's u, [width]
    __shared__ float red[HC_MAX_THREADS / 32];
    __shared__ float coef[S * S + 2 * S];   // mix, out, in
    const int tid = threadIdx.x, HC_THREADS = blockDim.x;
    const int64_t r = p.row_index ? p.row_index[blockIdx.x] : (int64_t)blockIdx.x;
    const bool write = p.y != nullptr, store = write && !p.row_index;
    for (int i = tid; i < S * S + 2 * S; i += HC_THREADS) {
        float c;
        if (i < S * S)
            c = p.mix ? p.mix[i] : (i / S == i % S ? 1.f : 0.f);
        else if (i < S * S + S)
            c = (p.out_coef ? p.out_coef[i - S * S] : 1.f) * p.mult;
        else
            c = p.in_coef ? p.in_coef[i - S * S - S] : 1.f;
        coef[i] = c;
    }
    __syncthreads();
    const float* mix = coef;
    const float* outc = coef + S * S;
    const float* inc = coef + S * S + S;
    float* x = p.streams + r * p.width;
    const float* y = write ? p.y + r * p.width : nullptr;
    float ss = 0.f;
    for (int c = tid; c < p.width; c += HC_THREADS) {
        float v[S];
#pragma unroll
        for (int s = 0; s < S; s++) v[s] = x[(int64_t)s * p.stream_stride + c];
        if (write) {
            const float yc = y[c];
            float nv[S];
#pragma unroll
            for (int t = 0; t < S; t++) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < S; s++) a = fmaf(mix[s * S + t], v[s], a);
                nv[t] = fmaf(outc[t], yc, a);
            }
#pragma unroll
            for (int t = 0; t < S; t++) {
                v[t] = nv[t];
                if (store) x[(int64_t)t * p.stream_stride + c] = nv[t];
            }
        }
        if (p.x_out) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < S; s++) u = fmaf(inc[s], v[s], u);
            u_s[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!p.x_out) return;
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < HC_THREADS / 32; i++) total += red[i];
    const float inv = 1.0f / sqrtf(total / (float)p.width + p.eps);
    TO* o = (TO*)p.x_out + (int64_t)blockIdx.x * p.width;
    for (int c = tid; c < p.width; c += HC_THREADS) o[c] = from_f32<TO>(u_s[c] * inv * p.norm_w[c]);
}

// streams[s][r, :] = float32(table[ids[r], :]) * scale for every stream s: all streams start as the embedding output
template <typename T>
__global__ void embed_streams_kernel(const T* __restrict__ table, const int* __restrict__ ids, int hidden, int vocab, float* __restrict__ streams,
                                     int64_t stream_stride, int n_streams, float scale) {
    const int r = blockIdx.x;
    int id = ids[r];
    if (!gb_check(id, vocab, GB_CHECK_TOKEN_ID) || id < 0 || id >= vocab) id = 0;   // ids are validated on the host
    const T* src = table + (int64_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_f32<T>(src[i]) * scale;   // scale 1 changes no bit
        for (int s = 0; s < n_streams; s++) streams[s * stream_stride + (int64_t)r * hidden + i] = v;
    }
}

template <typename TO, int S>
int launch_s(const HyperParams& p, cudaStream_t stream) {
    const size_t smem = p.x_out ? (size_t)p.width * sizeof(float) : 0;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) GB_REFUSE("hyper_mix_norm: rows of %d are wider than shared memory holds", p.width);
        cudaError_t e = cudaFuncSetAttribute(hyper_mix_norm_kernel<TO, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) GB_REFUSE("hyper_mix_norm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    // few rows: more threads a row, so that enough loads are in flight
    int threads = p.rows >= 1024 ? 256 : (p.rows >= 256 ? 512 : 1024);
    while (threads > 64 && threads > p.width) threads >>= 1;
    hyper_mix_norm_kernel<TO, S><<<p.rows, threads, smem, stream>>>(p);
    GB_CHECK_LAUNCH("hyper_mix_norm");
    return 0;
}

template <typename TO>
int launch(const HyperParams& p, cudaStream_t stream) {
    switch (p.n_streams) {
        case 1: return launch_s<TO, 1>(p, stream);
        case 2: return launch_s<TO, 2>(p, stream);
        case 3: return launch_s<TO, 3>(p, stream);
        case 4: return launch_s<TO, 4>(p, stream);
        case 5: return launch_s<TO, 5>(p, stream);
        case 6: return launch_s<TO, 6>(p, stream);
        case 7: return launch_s<TO, 7>(p, stream);
        case 8: return launch_s<TO, 8>(p, stream);
    }
    GB_REFUSE("hyper_mix_norm: %d streams; 1 to 8", p.n_streams);
}

}  // namespace

GB_API int gb_hyper_mix_norm(const HyperParams* pp, int out_dtype, cudaStream_t stream) {
    HyperParams p = *pp;
    if (p.rows <= 0) return 0;
    if (!p.streams || p.width <= 0) GB_REFUSE("hyper_mix_norm: no streams or width %d", p.width);
    if (!p.y && !p.x_out) GB_REFUSE("hyper_mix_norm: nothing to add and nothing to norm");
    if (p.x_out && !p.norm_w) GB_REFUSE("hyper_mix_norm: a normed output without a norm weight");
    if (p.row_index && !p.x_out) GB_REFUSE("hyper_mix_norm: rows picked by index are only read");
    if (out_dtype == GB_F32) return launch<float>(p, stream);
    if (out_dtype == GB_BF16) return launch<__nv_bfloat16>(p, stream);
    GB_REFUSE("hyper_mix_norm: unknown dtype %d", out_dtype);
}

GB_API int gb_embed_streams(const void* table, int table_dtype, const int* ids, int rows, int hidden, int vocab, float* streams,
                            int64_t stream_stride, int n_streams, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || vocab <= 0 || n_streams <= 0) GB_REFUSE("embed_streams: hidden %d, vocab %d, %d streams", hidden, vocab, n_streams);
    if (table_dtype == GB_F32)
        embed_streams_kernel<float><<<rows, 256, 0, stream>>>((const float*)table, ids, hidden, vocab, streams, stream_stride, n_streams, scale);
    else if (table_dtype == GB_BF16)
        embed_streams_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>((const __nv_bfloat16*)table, ids, hidden, vocab, streams, stream_stride,
                                                                      n_streams, scale);
    else
        GB_REFUSE("embed_streams: unknown table dtype %d", table_dtype);
    GB_CHECK_LAUNCH("embed_streams");
    return 0;
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_hyper)
