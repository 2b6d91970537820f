// Attention whose weights are not normalised over the keys, and the short convolution ahead of it.
//
// conv_qkv: per row, a causal convolution over time on every channel of the projected q | k | v
// (y_t = sum_j c[ch, j] u_(t - taps + 1 + j)), then each head divided by its root mean square (q and k,
// and v, each optional), q written to a buffer of its own and k and v into the paged cache.  The rows a
// tap reaches back to are the step's own rows of the same sequence or, before the step's first row, the
// sequence's state: its last taps - 1 projected rows, zero when the sequence starts, so that a prompt cut
// into steps and a token decoded alone see the same inputs.  conv_state_update then moves the state on.
//
// attention_sigmoid: out[i, h] = g(i, h) * sum_j sigmoid((q_i . k_j) * scale + b_h) v_j over the visible
// keys j <= i (i - j < window if there is one), g = sigmoid of the head's gate pre-activation if gates are
// given.  Scores, weights and sums are fp32.  A CTA owns one (sequence, kv head, tile of query rows) as
// the softmax kernel on the CUDA cores does; keys are visited in tiles of 32 that start at absolute
// positions 0, 32, 64, ..., and every weight is independent of the others, so a row's result does not
// depend on how its sequence was cut into steps or on what else is in the batch.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace {

constexpr int MAX_TAPS = 8;

template <typename T>
__global__ void __launch_bounds__(128) conv_qkv_kernel(ConvQkvParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = blockIdx.x;
    const int seq = p.row_seq[row], pos = p.row_pos[row];
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    const int t_in = (int)(row - p.seq_q_start[seq]);     // the row's place among its sequence's rows of this step
    const int taps = p.taps, back_max = taps > 0 ? taps - 1 : 0;
    const int qd = p.heads * p.d, kd = p.kv_heads * p.d;
    const T* base = (const T*)p.qkv;
    const float* state = p.state ? p.state + (int64_t)slot * p.state_slot_stride : nullptr;
    const int n_heads = p.heads + 2 * p.kv_heads;
    for (int hh = warp; hh < n_heads; hh += 4) {
        // which head: query heads, then key heads, then value heads
        int c0, n, kind;
        if (hh < p.heads)
            c0 = hh * p.d, n = p.d, kind = 0;
        else if (hh < p.heads + p.kv_heads)
            c0 = qd + (hh - p.heads) * p.d, n = p.d, kind = 1;
        else
            c0 = qd + kd + (hh - p.heads - p.kv_heads) * p.dv, n = p.dv, kind = 2;
        float y[8];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int i = lane + 32 * e;
            y[e] = 0.f;
            if (i >= n) continue;
            const int ch = c0 + i;
            if (taps <= 0) {
                y[e] = to_f32<T>(base[row * p.row_stride + ch]);
            } else {
                float a = 0.f;
                for (int j = 0; j < taps; j++) {
                    const int back = back_max - j;
                    float uv;
                    if (t_in - back >= 0)
                        uv = to_f32<T>(base[(row - back) * p.row_stride + ch]);
                    else
                        uv = state[(int64_t)(back_max + t_in - back) * p.channels + ch];
                    a = fmaf(p.conv_w[(int64_t)ch * taps + j], uv, a);
                }
                y[e] = a;
            }
            ss = fmaf(y[e], y[e], ss);
        }
        const bool normed = kind == 2 ? p.v_norm : p.qk_norm;
        float inv = 1.f;
        if (normed) inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + p.eps);
        T* dst;
        if (kind == 0) {
            dst = (T*)p.q_out + row * p.q_out_stride + c0;
        } else {
            const int* bt = block_table_row(p.block_table, p.bt_stride, slot, p.max_slots);
            const int64_t page = page_of(bt, pos, p.bt_stride, p.pages);
            const int kvh = kind == 1 ? hh - p.heads : hh - p.heads - p.kv_heads;
            const int64_t at = (page * p.kv_heads + kvh) * GB_PAGE + (pos % GB_PAGE);
            dst = kind == 1 ? (T*)p.k_plane + at * p.d : (T*)p.v_plane + at * p.dv;
        }
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int i = lane + 32 * e;
            if (i < n) dst[i] = from_f32<T>(y[e] * inv);
        }
    }
}

// the sequence's last taps - 1 projected rows after this step: from the step's rows, or, where the step
// brought fewer, from what the state held, moved up
template <typename T>
__global__ void conv_state_update_kernel(ConvQkvParams p) {
    const int seq = blockIdx.y;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= p.channels) return;
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    const int keep = p.taps - 1;
    const int q_len = p.seq_q_len[seq];
    const int64_t q_start = p.seq_q_start[seq];
    float* state = p.state + (int64_t)slot * p.state_slot_stride;
    const T* base = (const T*)p.qkv;
    float old[MAX_TAPS];
    for (int j = 0; j < keep; j++) old[j] = state[(int64_t)j * p.channels + ch];
    for (int j = 0; j < keep; j++) {
        const int t = q_len - keep + j;
        state[(int64_t)j * p.channels + ch] = t >= 0 ? to_f32<T>(base[(q_start + t) * p.row_stride + ch]) : old[j + q_len];
    }
}

constexpr int RW = 4;       // rows per warp
constexpr int ROWS = 16;    // rows per CTA (4 warps)
constexpr int KT = 32;      // keys per tile

template <typename T, int NE>
__global__ void __launch_bounds__(128) attn_sigmoid_kernel(SigmoidAttnParams p) {
    extern __shared__ float sm[];
    const int d = p.d, ks = d + 1;
    const int dv = p.dv > 0 ? p.dv : p.d, vs = dv + 1;
    float* Qs = sm;                // [16][d], pre-scaled
    float* Ks = Qs + ROWS * d;     // [32][d + 1]
    float* Vs = Ks + KT * ks;      // [32][dv + 1]

    const int G = p.heads / p.kv_heads;
    const int GC = G < ROWS ? G : ROWS;
    const int hchunks = (G + GC - 1) / GC;
    const int QT = ROWS / GC;

    const int seq = blockIdx.z;
    const int kvh = blockIdx.y / hchunks, chunk = blockIdx.y % hchunks;
    const int q_len = p.seq_q_len[seq], kv_len = p.seq_kv_len[seq];
    const int q0 = blockIdx.x * QT;
    if (q0 >= q_len) return;
    const int past = kv_len - q_len;
    const int q_start = p.seq_q_start[seq];
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int idx = tid; idx < ROWS * d; idx += 128) {
        int r = idx / d, c = idx - r * d;
        int qi = r / GC, hg = chunk * GC + r % GC;
        bool ok = qi < QT && q0 + qi < q_len && hg < G;
        float v = 0.f;
        if (ok) {
            const T* qp = (const T*)p.q + (int64_t)(q_start + q0 + qi) * p.q_row_stride + (int64_t)(kvh * G + hg) * d;
            v = to_f32<T>(qp[c]) * p.scale;
        }
        Qs[idx] = v;
    }

    int row_pos[RW], row_head[RW], row_q[RW];
    bool row_ok[RW];
    float row_bias[RW];
#pragma unroll
    for (int rr = 0; rr < RW; rr++) {
        int r = warp * RW + rr;
        int qi = r / GC, hg = chunk * GC + r % GC;
        row_ok[rr] = qi < QT && q0 + qi < q_len && hg < G;
        row_q[rr] = q0 + qi;
        row_head[rr] = kvh * G + hg;
        row_pos[rr] = past + q0 + qi;
        row_bias[rr] = (row_ok[rr] && p.score_bias) ? p.score_bias[row_head[rr]] : 0.f;
    }

    int last_q = (q0 + QT < q_len ? q0 + QT : q_len) - 1;
    const int hi_pos = past + last_q;
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = past + q0 - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    const int t_lo = lo_pos / KT, t_hi = hi_pos / KT + 1;

    float acc[RW][NE];
#pragma unroll
    for (int rr = 0; rr < RW; rr++)
#pragma unroll
        for (int e = 0; e < NE; e++) acc[rr][e] = 0.f;

    for (int t = t_lo; t < t_hi; t++) {
        __syncthreads();
        for (int jj = 0; jj < 8; jj++) {
            int j = warp * 8 + jj;
            int key = t * KT + j;
            if (key <= hi_pos) {
                int64_t page = page_of(bt, key, p.bt_stride, p.pages);
                int64_t at = (page * p.kv_heads + kvh) * GB_PAGE + (key % GB_PAGE);
                const T* kp = (const T*)p.k_plane + at * (int64_t)d;
                const T* vp = (const T*)p.v_plane + at * (int64_t)dv;
                for (int c = lane; c < d; c += 32) Ks[j * ks + c] = to_f32<T>(kp[c]);
                for (int c = lane; c < dv; c += 32) Vs[j * vs + c] = to_f32<T>(vp[c]);
            } else {
                for (int c = lane; c < d; c += 32) Ks[j * ks + c] = 0.f;
                for (int c = lane; c < dv; c += 32) Vs[j * vs + c] = 0.f;
            }
        }
        __syncthreads();

        float s[RW];
#pragma unroll
        for (int rr = 0; rr < RW; rr++) s[rr] = 0.f;
        const float* krow = Ks + lane * ks;
        const float* qrow = Qs + warp * RW * d;
        for (int c = 0; c < d; c++) {
            float kv = krow[c];
#pragma unroll
            for (int rr = 0; rr < RW; rr++) s[rr] = fmaf(qrow[rr * d + c], kv, s[rr]);
        }
        const int key = t * KT + lane;
        float pr[RW];
#pragma unroll
        for (int rr = 0; rr < RW; rr++) {
            bool valid = row_ok[rr] && key <= row_pos[rr] && (p.window <= 0 || key > row_pos[rr] - p.window);
            pr[rr] = valid ? 1.f / (1.f + expf(-(s[rr] + row_bias[rr]))) : 0.f;
        }
        for (int jj = 0; jj < KT; jj++) {
            const float* vrow = Vs + jj * vs;
#pragma unroll
            for (int rr = 0; rr < RW; rr++) {
                float pj = __shfl_sync(0xffffffffu, pr[rr], jj);
#pragma unroll
                for (int e = 0; e < NE; e++) {
                    int c = lane + 32 * e;
                    if (c < dv) acc[rr][e] = fmaf(pj, vrow[c], acc[rr][e]);
                }
            }
        }
    }

#pragma unroll
    for (int rr = 0; rr < RW; rr++) {
        if (!row_ok[rr]) continue;
        const int64_t row = q_start + row_q[rr];
        T* op = (T*)p.out + row * p.out_row_stride + (int64_t)row_head[rr] * dv;
        float g = 1.f;
        if (p.gate) g = 1.f / (1.f + expf(-to_f32<T>(((const T*)p.gate)[row * p.gate_stride + row_head[rr]])));
#pragma unroll
        for (int e = 0; e < NE; e++) {
            int c = lane + 32 * e;
            if (c < dv) op[c] = from_f32<T>(acc[rr][e] * g);
        }
    }
}

template <typename T, int NE>
int launch_ne(const SigmoidAttnParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_sigmoid_kernel<T, NE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) GB_REFUSE("attention_sigmoid: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attn_sigmoid_kernel<T, NE><<<grid, 128, smem, stream>>>(p);
    GB_CHECK_LAUNCH("attention_sigmoid");
    return 0;
}

template <typename T>
int launch(const SigmoidAttnParams& p, cudaStream_t stream) {
    const int G = p.heads / p.kv_heads;
    const int GC = G < ROWS ? G : ROWS;
    const int hchunks = (G + GC - 1) / GC;
    const int QT = ROWS / GC;
    dim3 grid(ceil_div(p.max_q_len, QT), p.kv_heads * hchunks, p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("attention_sigmoid: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    const int dv = p.dv > 0 ? p.dv : p.d;
    size_t smem = ((size_t)ROWS * p.d + (size_t)KT * (p.d + 1) + (size_t)KT * (dv + 1)) * sizeof(float);
    switch (ceil_div(dv, 32)) {
        case 1: return launch_ne<T, 1>(p, grid, smem, stream);
        case 2: return launch_ne<T, 2>(p, grid, smem, stream);
        case 3: return launch_ne<T, 3>(p, grid, smem, stream);
        case 4: return launch_ne<T, 4>(p, grid, smem, stream);
        case 5: return launch_ne<T, 5>(p, grid, smem, stream);
        case 6: return launch_ne<T, 6>(p, grid, smem, stream);
        case 7: return launch_ne<T, 7>(p, grid, smem, stream);
        case 8: return launch_ne<T, 8>(p, grid, smem, stream);
    }
    GB_REFUSE("attention_sigmoid: value size %d is larger than 256", dv);
}

template <typename T>
int launch_conv(const ConvQkvParams& p, cudaStream_t stream) {
    conv_qkv_kernel<T><<<p.rows, 128, 0, stream>>>(p);
    GB_CHECK_LAUNCH("conv_qkv");
    if (p.taps > 1) {
        dim3 grid(ceil_div(p.channels, 128), p.nseq);
        if (grid.y > 65535) GB_REFUSE("conv_qkv: %d sequences exceed one launch", p.nseq);
        conv_state_update_kernel<T><<<grid, 128, 0, stream>>>(p);
        GB_CHECK_LAUNCH("conv_state_update");
    }
    return 0;
}

}  // namespace

GB_API int gb_conv_qkv(const ConvQkvParams* pp, int dtype, cudaStream_t stream) {
    ConvQkvParams p = *pp;
    if (p.rows <= 0 || p.nseq <= 0) return 0;
    if (p.heads <= 0 || p.kv_heads <= 0 || p.d <= 0 || p.d > 256 || p.dv <= 0 || p.dv > 256)
        GB_REFUSE("conv_qkv: %d + %d heads of %d / %d channels", p.heads, p.kv_heads, p.d, p.dv);
    if (p.taps < 0 || p.taps > MAX_TAPS) GB_REFUSE("conv_qkv: %d taps; at most %d", p.taps, MAX_TAPS);
    if (p.channels != (p.heads + p.kv_heads) * p.d + p.kv_heads * p.dv) GB_REFUSE("conv_qkv: %d channels do not fit the heads", p.channels);
    if (p.taps > 0 && !p.conv_w) GB_REFUSE("conv_qkv: taps without weights");
    if (p.taps > 1 && (!p.state || p.state_slot_stride < (int64_t)(p.taps - 1) * p.channels)) GB_REFUSE("conv_qkv: the state has no room for %d rows", p.taps - 1);
    if (!p.qkv || !p.q_out || !p.k_plane || !p.v_plane) GB_REFUSE("conv_qkv: a tensor is missing");
    if (dtype == GB_F32) return launch_conv<float>(p, stream);
    if (dtype == GB_BF16) return launch_conv<__nv_bfloat16>(p, stream);
    GB_REFUSE("conv_qkv: unknown dtype %d", dtype);
}

GB_API int gb_attention_sigmoid(const SigmoidAttnParams* pp, int dtype, cudaStream_t stream) {
    SigmoidAttnParams p = *pp;
    if (p.nseq <= 0 || p.max_q_len <= 0) return 0;
    if (p.heads <= 0 || p.kv_heads <= 0 || p.heads % p.kv_heads) GB_REFUSE("attention: %d heads over %d kv heads", p.heads, p.kv_heads);
    if (p.d <= 0 || p.d > 256) GB_REFUSE("attention_sigmoid: head_dim %d is outside [1, 256]", p.d);
    if (p.window < 0) GB_REFUSE("attention: window %d", p.window);
    if (p.dv < 0 || p.dv > 256) GB_REFUSE("attention_sigmoid: value size %d is outside [1, 256]", p.dv);
    if (dtype == GB_F32) return launch<float>(p, stream);
    if (dtype == GB_BF16) return launch<__nv_bfloat16>(p, stream);
    GB_REFUSE("attention: unknown dtype %d", dtype);
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_attention_sigmoid)
