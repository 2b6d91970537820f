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
//
// In bfloat16, with key and value heads of whole 16s up to 128, the same sum runs on mma.sync tensor cores:
// a CTA owns 64 query rows of one head of one sequence (16 rows a warp) and walks the pages its rows can see,
// a page of 64 keys fetched with cp.async one page ahead of the arithmetic; the weights are formed in fp32
// from the fp32 scores, rounded to bfloat16 for the second product (the values are bfloat16), and summed in
// fp32.  Prompts, portions and single tokens take the same kernel.
#include "api.h"
#include "mma.cuh"

#include <math.h>

namespace {

constexpr int MAX_TAPS = 16;
typedef __nv_bfloat16 bf16;

// sigmoid(z) for z given as half its argument: 0.5 + 0.5 tanh(z / 2), one special-function instruction; its error
// (about 2^-11 relative) is below the rounding of the weight to bfloat16 that follows
__device__ __forceinline__ float sigmoid_of_half(float half_z) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(half_z));
    return fmaf(t, 0.5f, 0.5f);
}

// copy 64 rows of N bf16 (contiguous in global memory) into padded shared rows
template <int N>
__device__ __forceinline__ void load_page(bf16* dst, const bf16* src, int tid, int nthreads) {
    constexpr int SD = N + 8, CH = N / 8;
    for (int idx = tid; idx < 64 * CH; idx += nthreads) {
        int row = idx / CH, c = idx - row * CH;
        cp_async16(dst + row * SD + c * 8, src + row * N + c * 8, 16);
    }
}

template <int HD, int DV>
__global__ void __launch_bounds__(128) attn_sigmoid_mma_kernel(SigmoidAttnParams p) {
    constexpr int SD = HD + 8, SV = DV + 8, KS = HD / 16, NF = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + 64 * SD;
    bf16* Vs = Ks + 2 * 64 * SD;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int q_len = p.seq_q_len[seq], kv_len = p.seq_kv_len[seq];
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;  // late (long) tiles first
    const int q0 = qt * 64;
    if (q0 >= q_len) return;
    const int past = kv_len - q_len;
    const int q_start = p.seq_q_start[seq];
    const int G = p.heads / p.kv_heads, kvh = head / G;
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);
    const bf16* kbase = (const bf16*)p.k_plane;
    const bf16* vbase = (const bf16*)p.v_plane;

    {
        constexpr int CH = HD / 8;
        const bf16* qsrc = (const bf16*)p.q + (int64_t)(q_start + q0) * p.q_row_stride + (int64_t)head * HD;
        for (int idx = tid; idx < 64 * CH; idx += 128) {
            int row = idx / CH, c = idx - row * CH;
            bool ok = q0 + row < q_len;
            cp_async16(Qs + row * SD + c * 8, ok ? qsrc + (int64_t)row * p.q_row_stride + c * 8 : qsrc, ok ? 16 : 0);
        }
    }
    const int last_q = (q0 + 64 < q_len ? q0 + 64 : q_len) - 1;
    const int hi_pos = past + last_q;
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = past + q0 - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    const int t_lo = lo_pos / 64, t_hi = hi_pos / 64;
    const int n_tiles = t_hi - t_lo + 1;

    auto load_tile = [&](int t, int buf) {
        int64_t page = page_of(bt, t * 64, p.bt_stride, p.pages);
        int64_t at = (page * p.kv_heads + kvh) * 64;
        load_page<HD>(Ks + buf * 64 * SD, kbase + at * HD, tid, 128);
        load_page<DV>(Vs + buf * 64 * SV, vbase + at * DV, tid, 128);
    };
    load_tile(t_lo, 0);
    cp_async_commit();

    const float sc = 0.5f * p.scale;                                  // half the argument of the sigmoid: see sigmoid_of_half
    const float bias = 0.5f * (p.score_bias ? p.score_bias[head] : 0.f);
    const int row0 = past + q0 + warp * 16 + g;  // absolute position of this thread's first row
    const int row1 = row0 + 8;
    float o[NF][4];
#pragma unroll
    for (int j = 0; j < NF; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
    uint32_t qf[KS][4];

    for (int ti = 0; ti < n_tiles; ti++) {
        const int t = t_lo + ti;
        const int buf = ti & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (ti + 1 < n_tiles) load_tile(t + 1, buf ^ 1);
        cp_async_commit();
        if (ti == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
                ldmatrix_x4(qf[ks], Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks * 16 + (lane >> 4) * 8);
        }
        const bf16* kt = Ks + buf * 64 * SD;
        const bf16* vt = Vs + buf * 64 * SV;
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + (jp * 16 + (lane & 7) + (lane >> 4) * 8) * SD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(s[jp * 2], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b[0], b[1]);
                mma_bf16_16816(s[jp * 2 + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b[2], b[3]);
            }
        }
        // the weights: sigmoid(score * scale + bias) where the key is visible, by absolute position; a tile that
        // every row of this warp sees whole needs no masks
        const int wrow_lo = past + q0 + warp * 16, wrow_hi = wrow_lo + 15;
        const bool whole = t * 64 + 63 <= wrow_lo && (p.window <= 0 || t * 64 > wrow_hi - p.window);
        uint32_t pa[4][4];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                w[e] = sigmoid_of_half(fmaf(s[j][e], sc, bias));
                if (!whole) {
                    int key = t * 64 + j * 8 + t4 * 2 + (e & 1);
                    int row = (e & 2) ? row1 : row0;
                    bool ok = key <= row && (p.window <= 0 || key > row - p.window);
                    w[e] = ok ? w[e] : 0.f;
                }
            }
            pa[j >> 1][(j & 1) * 2] = pack_bf16(w[0], w[1]);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(w[2], w[3]);
        }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
#pragma unroll
            for (int c = 0; c < DV / 16; c++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SV + c * 16 + (lane >> 4) * 8);
                mma_bf16_16816(o[c * 2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[0], b[1]);
                mma_bf16_16816(o[c * 2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
    bf16* ob = (bf16*)p.out + (int64_t)head * DV;
    const bf16* gate = (const bf16*)p.gate;
    if (r0 < q_len) {
        const int64_t row = q_start + r0;
        const float gv = gate ? 1.f / (1.f + expf(-__bfloat162float(gate[row * p.gate_stride + head]))) : 1.f;
        bf16* op = ob + row * p.out_row_stride;
#pragma unroll
        for (int j = 0; j < NF; j++) *reinterpret_cast<uint32_t*>(op + j * 8 + t4 * 2) = pack_bf16(o[j][0] * gv, o[j][1] * gv);
    }
    if (r1 < q_len) {
        const int64_t row = q_start + r1;
        const float gv = gate ? 1.f / (1.f + expf(-__bfloat162float(gate[row * p.gate_stride + head]))) : 1.f;
        bf16* op = ob + row * p.out_row_stride;
#pragma unroll
        for (int j = 0; j < NF; j++) *reinterpret_cast<uint32_t*>(op + j * 8 + t4 * 2) = pack_bf16(o[j][2] * gv, o[j][3] * gv);
    }
}

// Single tokens: a CTA owns one (sequence, kv head); the 16 rows of its tiles are the query heads of the group,
// so the group's heads share every key and value that is read.  The four warps take 16 keys each of every page
// and keep sums of their own, which meet in shared memory at the end (the weights are not normalised: the sums
// simply add).
template <int HD, int DV>
__global__ void __launch_bounds__(128) attn_sigmoid_decode_mma_kernel(SigmoidAttnParams p) {
    constexpr int SD = HD + 8, SV = DV + 8, KS = HD / 16, NF = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);      // [16][SD]
    bf16* Ks = Qs + 16 * SD;                           // [2][64][SD]
    bf16* Vs = Ks + 2 * 64 * SD;                       // [2][64][SV]
    float* red = reinterpret_cast<float*>(Vs + 2 * 64 * SV);   // [4][16][DV + 1]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.y, kvh = blockIdx.x;
    const int G = p.heads / p.kv_heads;
    const int pos = p.seq_kv_len[seq] - 1;             // the token's position
    const int64_t row = p.seq_q_start[seq];
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);
    const bf16* kbase = (const bf16*)p.k_plane;
    const bf16* vbase = (const bf16*)p.v_plane;
    {
        constexpr int CH = HD / 8;
        const bf16* qsrc = (const bf16*)p.q + row * p.q_row_stride + (int64_t)kvh * G * HD;
        for (int idx = tid; idx < 16 * CH; idx += 128) {
            int r = idx / CH, c = idx - r * CH;
            bool ok = r < G;
            cp_async16(Qs + r * SD + c * 8, ok ? qsrc + (int64_t)r * HD + c * 8 : qsrc, ok ? 16 : 0);
        }
    }
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = pos - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    const int t_lo = lo_pos / 64, t_hi = pos / 64;
    const int n_tiles = t_hi - t_lo + 1;
    auto load_tile = [&](int t, int buf) {
        int64_t page = page_of(bt, t * 64, p.bt_stride, p.pages);
        int64_t at = (page * p.kv_heads + kvh) * 64;
        load_page<HD>(Ks + buf * 64 * SD, kbase + at * HD, tid, 128);
        load_page<DV>(Vs + buf * 64 * SV, vbase + at * DV, tid, 128);
    };
    load_tile(t_lo, 0);
    cp_async_commit();

    const float sc = 0.5f * p.scale;
    const int h0 = kvh * G + g, h1 = h0 + 8;           // the heads of this thread's two rows
    const float bias0 = 0.5f * (p.score_bias && g < G ? p.score_bias[h0] : 0.f);
    const float bias1 = 0.5f * (p.score_bias && g + 8 < G ? p.score_bias[h1] : 0.f);
    float o[NF][4];
#pragma unroll
    for (int j = 0; j < NF; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
    uint32_t qf[KS][4];
    for (int ti = 0; ti < n_tiles; ti++) {
        const int t = t_lo + ti;
        const int buf = ti & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (ti + 1 < n_tiles) load_tile(t + 1, buf ^ 1);
        cp_async_commit();
        if (ti == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ks++) ldmatrix_x4(qf[ks], Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks * 16 + (lane >> 4) * 8);
        }
        const bf16* kt = Ks + buf * 64 * SD;
        const bf16* vt = Vs + buf * 64 * SV;
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            uint32_t b[4];
            ldmatrix_x4(b, kt + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * SD + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16_16816(s[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b[0], b[1]);
            mma_bf16_16816(s[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b[2], b[3]);
        }
        uint32_t pa[4];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = t * 64 + warp * 16 + j * 8 + t4 * 2 + (e & 1);
                const bool ok = key <= pos && (p.window <= 0 || key > pos - p.window);
                w[e] = ok ? sigmoid_of_half(fmaf(s[j][e], sc, (e & 2) ? bias1 : bias0)) : 0.f;
            }
            pa[j * 2] = pack_bf16(w[0], w[1]);
            pa[j * 2 + 1] = pack_bf16(w[2], w[3]);
        }
#pragma unroll
        for (int c = 0; c < DV / 16; c++) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vt + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SV + c * 16 + (lane >> 4) * 8);
            mma_bf16_16816(o[c * 2], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
            mma_bf16_16816(o[c * 2 + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    // the four warps' sums, in warp order
#pragma unroll
    for (int j = 0; j < NF; j++) {
        float* r0 = red + ((warp * 16 + g) * (DV + 1)) + j * 8 + t4 * 2;
        float* r1 = red + ((warp * 16 + g + 8) * (DV + 1)) + j * 8 + t4 * 2;
        r0[0] = o[j][0], r0[1] = o[j][1], r1[0] = o[j][2], r1[1] = o[j][3];
    }
    __syncthreads();
    const bf16* gate = (const bf16*)p.gate;
    for (int idx = tid; idx < G * DV; idx += 128) {
        const int r = idx / DV, c = idx - r * DV;
        const int head = kvh * G + r;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) a += red[(w * 16 + r) * (DV + 1) + c];
        if (gate) a *= 1.f / (1.f + expf(-__bfloat162float(gate[row * p.gate_stride + head])));
        ((bf16*)p.out)[row * p.out_row_stride + (int64_t)head * DV + c] = __float2bfloat16_rn(a);
    }
}

template <int HD, int DV>
int launch_mma_dv(const SigmoidAttnParams& p, cudaStream_t stream) {
    if (p.max_q_len == 1 && p.heads / p.kv_heads <= 16) {
        const size_t dsmem = (size_t)(16 * (HD + 8) + 2 * 64 * (HD + 8) + 2 * 64 * (DV + 8)) * sizeof(bf16) + (size_t)4 * 16 * (DV + 1) * sizeof(float);
        static bool dconfigured = false;
        if (!dconfigured && dsmem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(attn_sigmoid_decode_mma_kernel<HD, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsmem);
            if (e != cudaSuccess) GB_REFUSE("attention_sigmoid: cannot reserve %zu bytes of shared memory: %s", dsmem, cudaGetErrorString(e));
            dconfigured = true;
        }
        dim3 dgrid(p.kv_heads, p.nseq);
        if (dgrid.y > 65535) GB_REFUSE("attention_sigmoid: %d sequences exceed one launch", p.nseq);
        attn_sigmoid_decode_mma_kernel<HD, DV><<<dgrid, 128, dsmem, stream>>>(p);
        GB_CHECK_LAUNCH("attention_sigmoid_decode_mma");
        return 0;
    }
    const size_t smem = (size_t)(3 * 64 * (HD + 8) + 2 * 64 * (DV + 8)) * sizeof(bf16);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_sigmoid_mma_kernel<HD, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) GB_REFUSE("attention_sigmoid: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(ceil_div(p.max_q_len, 64), p.heads, p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("attention_sigmoid: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    attn_sigmoid_mma_kernel<HD, DV><<<grid, 128, smem, stream>>>(p);
    GB_CHECK_LAUNCH("attention_sigmoid_mma");
    return 0;
}

template <int HD>
int launch_mma(const SigmoidAttnParams& p, int dv, cudaStream_t stream) {
    switch (dv) {
        case 32: return launch_mma_dv<HD, 32>(p, stream);
        case 48: return launch_mma_dv<HD, 48>(p, stream);
        case 64: return launch_mma_dv<HD, 64>(p, stream);
        case 128: return launch_mma_dv<HD, 128>(p, stream);
    }
    return 1;
}

// whether the tensor-core kernel takes these sizes and pointers
bool mma_takes(const SigmoidAttnParams& p, int dv) {
    const bool hd = p.d == 32 || p.d == 64 || p.d == 96 || p.d == 128;
    const bool vd = dv == 32 || dv == 48 || dv == 64 || dv == 128;
    return hd && vd && !(p.q_row_stride & 7) && !((uintptr_t)p.q & 15) && !(p.out_row_stride & 1) && !((uintptr_t)p.out & 3);
}

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
    const bool move_state = taps > 1 && p.max_q_len == 1;     // single tokens: this thread also moves its channels' state on
    for (int hh = blockIdx.y * 4 + warp; hh < n_heads; hh += 4 * gridDim.y) {
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
                    // the value tap j read is what the state's row j - 1 holds after this token
                    if (move_state && j > 0) p.state[(int64_t)slot * p.state_slot_stride + (int64_t)(j - 1) * p.channels + ch] = uv;
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
    const int n_heads = p.heads + 2 * p.kv_heads;
    int chunks = 1;                       // few rows: the heads of a row are spread over several CTAs
    while (chunks * 4 < n_heads && p.rows * chunks < 296) chunks++;
    conv_qkv_kernel<T><<<dim3(p.rows, chunks), 128, 0, stream>>>(p);
    GB_CHECK_LAUNCH("conv_qkv");
    if (p.taps > 1 && p.max_q_len != 1) {
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

int gb_attention_sigmoid_tc5(const SigmoidAttnParams* pp, int rows, int pages, cudaStream_t stream);

// rows: packed query rows in the q buffer (the tcgen05 kernel's tensor map spans them); 0: not known
GB_API int gb_attention_sigmoid(const SigmoidAttnParams* pp, int dtype, int rows, cudaStream_t stream) {
    SigmoidAttnParams p = *pp;
    if (p.nseq <= 0 || p.max_q_len <= 0) return 0;
    if (p.heads <= 0 || p.kv_heads <= 0 || p.heads % p.kv_heads) GB_REFUSE("attention: %d heads over %d kv heads", p.heads, p.kv_heads);
    if (p.d <= 0 || p.d > 256) GB_REFUSE("attention_sigmoid: head_dim %d is outside [1, 256]", p.d);
    if (p.window < 0) GB_REFUSE("attention: window %d", p.window);
    if (p.dv < 0 || p.dv > 256) GB_REFUSE("attention_sigmoid: value size %d is outside [1, 256]", p.dv);
    if (dtype == GB_F32) return launch<float>(p, stream);
    const int dv = p.dv > 0 ? p.dv : p.d;
    // prompts of heads of 128: the tcgen05 kernel, as for the softmax (num_splits -2 asks for mma.sync instead)
    if (dtype == GB_BF16 && p.num_splits == 1 && p.d == 128 && dv == 128 && rows > 0 && p.max_q_len >= 65 && !((uintptr_t)p.q & 15) &&
        !(p.q_row_stride & 7) && !((uintptr_t)p.out & 15) && !(p.out_row_stride & 7)) {
        p.dv = 0;
        return gb_attention_sigmoid_tc5(&p, rows, p.pages, stream);
    }
    if (p.num_splits == -2) p.num_splits = 1;
    if (dtype == GB_BF16 && p.num_splits != -1 && mma_takes(p, dv)) {     // num_splits -1 asks for the CUDA-core kernel
        switch (p.d) {
            case 32: return launch_mma<32>(p, dv, stream);
            case 64: return launch_mma<64>(p, dv, stream);
            case 96: return launch_mma<96>(p, dv, stream);
            case 128: return launch_mma<128>(p, dv, stream);
        }
    }
    if (dtype == GB_BF16) return launch<__nv_bfloat16>(p, stream);
    GB_REFUSE("attention: unknown dtype %d", dtype);
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_attention_sigmoid)
