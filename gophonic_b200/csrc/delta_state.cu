// The generalized delta rule: a matrix state per (sequence, head), d key channels x dv value channels,
// fp32, updated for every token with a decay w and a removal rate a per key channel and the unit key
// u = k / sqrt(|k|^2 + key_eps):
//
//     S <- diag(w) S - (a * u) (u^T S) + k v^T          (both terms read the old S)
//     o = S^T r
//
// Columns of S are independent of one another, so the work is spread over (sequence, head, block of 16
// value columns) as in the decayed-state scan; what is new is that a token needs a sum over all key
// channels of the old state before the state can move on.  Both sums a token needs are taken of the old
// state in one pass, p1 = S^T u and p2 = S^T (w * r), and the output follows without a second sum:
//
//     o = p2 - (au . r) p1 + (k . r) v          with au = a * u,
//
// where the two dot products are per (token, head) numbers that the preparation kernel leaves behind.
// That kernel also turns the pre-activations into w = exp(-decay_scale * sigmoid(z_w + w0)) and
// a = sigmoid(z_a + b) and takes the keys' lengths, all in fp32; r, k and v are read as the projection left
// them.  A step of single tokens needs no preparation kernel: its one kernel prepares the token itself.
// The recurrence runs token by token, in order, for prompts and single tokens alike: the state after a
// token is the same bits however the sequence was cut into steps and whatever else the batch holds.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace {

constexpr int COLS = 16;     // value columns per CTA of the single-token kernel
constexpr int SLICES = 8;    // its slices of the key channels
constexpr int TT = 8;        // tokens staged at a time
constexpr int THREADS = 128;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

__global__ void tanh_kernel(float* __restrict__ z, int rows, int cols, int64_t stride) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * cols) return;
    float* at = z + (i / cols) * stride + i % cols;
    *at = tanhf(*at);
}

template <typename TW>
__device__ __forceinline__ float dot_row(const TW* __restrict__ w, const float* __restrict__ x, int n);
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ w, const float* __restrict__ x, int n) {
    float a = 0.f;
    for (int j = 0; j < n; j++) a = fmaf(w[j], x[j], a);
    return a;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int n) {
    float a = 0.f;
    if (!(n & 7) && !((uintptr_t)w & 15)) {
        for (int j = 0; j < n; j += 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(w + j);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                a = fmaf(__low2float(h[e]), x[j + 2 * e], a);
                a = fmaf(__high2float(h[e]), x[j + 2 * e + 1], a);
            }
        }
        return a;
    }
    for (int j = 0; j < n; j++) a = fmaf(__bfloat162float(w[j]), x[j], a);
    return a;
}

// ------------------------------------------------------------------------------------------
// preparation, one warp per (row, head): decay and removal rate from their pre-activations (in place; the
// removal rate is left multiplied by the unit key), and the token's numbers: (a u) . r, k . r and 1 / |k|.
template <typename T>
__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaStateParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = blockIdx.x;
    const int h = blockIdx.y * 4 + warp;
    if (h >= p.heads) return;
    const int d = p.d;
    const T* base = (const T*)p.rkv + row * p.row_stride;
    const T* r = base + p.r_off + h * d;
    const T* k = base + p.k_off + h * d;
    float* wz = p.decay + row * p.decay_stride + h * d;
    float* az = p.remove + row * p.remove_stride + h * d;
    float kk = 0.f;
    for (int c = lane; c < d; c += 32) {
        const float kv = to_f32<T>(k[c]);
        kk = fmaf(kv, kv, kk);
    }
    const float inv = 1.0f / sqrtf(warp_sum(kk) + p.key_eps);
    float aur = 0.f, kr = 0.f;
    for (int c = lane; c < d; c += 32) {
        const float kv = to_f32<T>(k[c]), rv = to_f32<T>(r[c]);
        const float a = sigmoid_f(az[c] + (p.remove_bias ? p.remove_bias[h * d + c] : 0.f));
        const float w = expf(-p.decay_scale * sigmoid_f(wz[c] + (p.decay_bias ? p.decay_bias[h * d + c] : 0.f)));
        const float au = a * (kv * inv);
        wz[c] = w;
        az[c] = au;
        aur = fmaf(au, rv, aur);
        kr = fmaf(kv, rv, kr);
    }
    aur = warp_sum(aur);
    kr = warp_sum(kr);
    if (lane == 0) *reinterpret_cast<float4*>(p.dots + (row * p.heads + h) * 4) = make_float4(aur, kr, inv, 0.f);
}

// ------------------------------------------------------------------------------------------
// the scan.  SLICES: slices of the key channels (8 or 16); RC: key channels per slice (a multiple of 4,
// RC * SLICES >= d).  A warp owns 32 / SLICES columns and its groups of lanes a slice of the key channels each; a
// thread keeps its RC state elements in registers across all tokens of the step.  8 slices are what is
// launched: a prompt of one sequence and 16 heads of 128 x 128 leaves schedulers without a warp, but 16 slices
// (twice the warps, each with half the state and one more exchange step a sum) measured 0.66 ms against 0.55,
// and a warp a column with 32 slices 0.74: the exchange steps a token's update waits for cost more than the
// idle schedulers.  A tile's rows are fetched into registers while the tile before it is
// worked on, and put into shared memory between two barriers.  With u = k / |k| the sum along the unit key
// is (S^T k) / |k|, so the keys themselves are staged and the token's 1 / |k| multiplies the finished sum.
template <typename T, int RC, int SLICES>
__global__ void __launch_bounds__(THREADS) delta_scan_kernel(DeltaStateParams p) {
    constexpr int COLS = 4 * (32 / SLICES);         // value columns per CTA: 16 with 8 slices, 8 with 16
    constexpr int P = (RC / 4) % 2 ? RC : RC + 4;   // slice stride in floats: P / 4 odd, so the 8 slices' 16-byte reads miss each other's banks
    constexpr int ROW = SLICES * P;
    extern __shared__ __align__(16) float smem[];
    float* rw_s = smem;                     // [TT][ROW]  w * r
    float* k_s = rw_s + TT * ROW;
    float* au_s = k_s + TT * ROW;           // a * u
    float* w_s = au_s + TT * ROW;
    float* v_s = w_s + TT * ROW;            // [TT][COLS]
    float* o_s = v_s + TT * COLS;           // [TT][COLS]
    float* dot_s = o_s + TT * COLS;         // [TT][4]
    float* st_s = dot_s + TT * 4;           // [SLICES * RC][COLS + 1]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slice = lane & (SLICES - 1), col = warp * (32 / SLICES) + lane / SLICES;
    const int d = p.d, dv = p.dv, H = p.heads;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int j0 = blockIdx.x * COLS;
    const int q_len = p.seq_q_len[seq], q_start = p.seq_q_start[seq];
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    float* S = p.state + (int64_t)slot * p.slot_stride + (int64_t)h * p.head_stride;

    for (int idx = tid; idx < SLICES * RC * COLS; idx += THREADS) {
        const int c = idx / COLS, jj = idx % COLS;
        st_s[c * (COLS + 1) + jj] = (c < d && j0 + jj < dv) ? S[(int64_t)c * dv + j0 + jj] : 0.f;
    }
    __syncthreads();
    float st[RC];
#pragma unroll
    for (int i = 0; i < RC; i++) st[i] = st_s[(slice * RC + i) * (COLS + 1) + col];

    const T* base = (const T*)p.rkv;
    constexpr int PER = TT * SLICES * RC / THREADS;   // elements of each staged array a thread fetches per tile
    // Every load of a fetch is unconditional (indices clamped into the tile) and nothing is done with the
    // values until they are stored: they are all in flight at once.  What lies outside the tile or the head
    // is replaced when it is stored: a token or channel that is not there changes nothing (decay 1, keys 0).
    T rr[PER], rk[PER], rv = from_f32<T>(0.f);
    float rw[PER], rau[PER], rdot = 0.f;
    auto fetch = [&](int t0) {
        const int nt = q_len - t0 < TT ? q_len - t0 : TT;
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = tid + e * THREADS;
            int t = idx / (SLICES * RC), c = idx % (SLICES * RC);
            t = t < nt ? t : nt - 1;
            c = c < d ? c : d - 1;
            const int64_t row = q_start + t0 + t;
            const T* rp = base + row * p.row_stride;
            rr[e] = rp[p.r_off + h * d + c];
            rk[e] = rp[p.k_off + h * d + c];
            rw[e] = p.decay[row * p.decay_stride + h * d + c];
            rau[e] = p.remove[row * p.remove_stride + h * d + c];
        }
        if (tid < TT * COLS) {
            int t = tid / COLS, jj = j0 + tid % COLS;
            t = t < nt ? t : nt - 1;
            jj = jj < dv ? jj : dv - 1;
            rv = base[(int64_t)(q_start + t0 + t) * p.row_stride + p.v_off + h * dv + jj];
        }
        if (tid < TT * 4) {
            int t = tid >> 2;
            t = t < nt ? t : nt - 1;
            rdot = p.dots[((int64_t)(q_start + t0 + t) * H + h) * 4 + (tid & 3)];
        }
    };
    if (q_len > 0) fetch(0);
    for (int t0 = 0; t0 < q_len; t0 += TT) {
        const int nt = q_len - t0 < TT ? q_len - t0 : TT;
        __syncthreads();   // the tile before is done with
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = tid + e * THREADS;
            const int t = idx / (SLICES * RC), c = idx % (SLICES * RC);
            const int at = t * ROW + (c / RC) * P + c % RC;
            const bool there = t < nt && c < d;
            rw_s[at] = there ? to_f32<T>(rr[e]) * rw[e] : 0.f;
            k_s[at] = there ? to_f32<T>(rk[e]) : 0.f;
            au_s[at] = there ? rau[e] : 0.f;
            w_s[at] = there ? rw[e] : 1.f;
        }
        if (tid < TT * COLS) {
            const int t = tid / COLS, jj = tid % COLS;
            v_s[tid] = (t < nt && j0 + jj < dv) ? to_f32<T>(rv) : 0.f;
        }
        if (tid < TT * 4) dot_s[tid] = (tid >> 2) < nt ? rdot : 0.f;
        __syncthreads();
        if (t0 + TT < q_len) fetch(t0 + TT);
        // all eight tokens of the tile, unrolled; a tile's missing tokens leave the state as it is
#pragma unroll
        for (int t = 0; t < TT; t++) {
            const float vj = v_s[t * COLS + col];
            const float* rwp = rw_s + t * ROW + slice * P;
            const float* kp = k_s + t * ROW + slice * P;
            float p1a = 0.f, p1b = 0.f, p2a = 0.f, p2b = 0.f;
#pragma unroll
            for (int i = 0; i < RC; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kp + i);
                const float4 r4 = *reinterpret_cast<const float4*>(rwp + i);
                p1a = fmaf(k4.x, st[i], p1a);
                p1b = fmaf(k4.y, st[i + 1], p1b);
                p1a = fmaf(k4.z, st[i + 2], p1a);
                p1b = fmaf(k4.w, st[i + 3], p1b);
                p2a = fmaf(r4.x, st[i], p2a);
                p2b = fmaf(r4.y, st[i + 1], p2b);
                p2a = fmaf(r4.z, st[i + 2], p2a);
                p2b = fmaf(r4.w, st[i + 3], p2b);
            }
            float p1 = p1a + p1b, p2 = p2a + p2b;
#pragma unroll
            for (int o = 1; o < SLICES; o <<= 1) {
                p1 += __shfl_xor_sync(0xffffffffu, p1, o);
                p2 += __shfl_xor_sync(0xffffffffu, p2, o);
            }
            p1 *= dot_s[4 * t + 2];        // along the unit key
            const float* au = au_s + t * ROW + slice * P;
            const float* ww = w_s + t * ROW + slice * P;
#pragma unroll
            for (int i = 0; i < RC; i += 4) {
                const float4 a4 = *reinterpret_cast<const float4*>(au + i);
                const float4 k4 = *reinterpret_cast<const float4*>(kp + i);
                const float4 w4 = *reinterpret_cast<const float4*>(ww + i);
                st[i] = fmaf(w4.x, st[i], fmaf(k4.x, vj, -a4.x * p1));
                st[i + 1] = fmaf(w4.y, st[i + 1], fmaf(k4.y, vj, -a4.y * p1));
                st[i + 2] = fmaf(w4.z, st[i + 2], fmaf(k4.z, vj, -a4.z * p1));
                st[i + 3] = fmaf(w4.w, st[i + 3], fmaf(k4.w, vj, -a4.w * p1));
            }
            if (slice == 0) o_s[t * COLS + col] = p2 - dot_s[4 * t] * p1 + dot_s[4 * t + 1] * vj;
        }
        __syncthreads();
        for (int idx = tid; idx < nt * COLS; idx += THREADS) {
            const int t = idx / COLS, jj = idx % COLS;
            if (j0 + jj < dv) p.out[(int64_t)(q_start + t0 + t) * p.out_stride + h * dv + j0 + jj] = o_s[idx];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RC; i++) st_s[(slice * RC + i) * (COLS + 1) + col] = st[i];
    __syncthreads();
    for (int idx = tid; idx < SLICES * RC * COLS; idx += THREADS) {
        const int c = idx / COLS, jj = idx % COLS;
        if (c < d && j0 + jj < dv) S[(int64_t)c * dv + j0 + jj] = st_s[c * (COLS + 1) + jj];
    }
}

// ------------------------------------------------------------------------------------------
// One token for every sequence (a decode step): the work is reading and writing the state once.  A CTA
// owns 16 columns of one head's S; thread (group g of 8, column j of 16) takes the channels g, g + 8, ...
// so that a warp's loads are whole 64-byte rows and keeps them in registers from load to store; the
// eight groups' partial sums meet in shared memory.  The CTA prepares the token itself (decay, removal
// rate, the key's length, the two dot products: a thread a channel, sums over the CTA), and with `low` and
// `w2` also the decay's pre-activation, z = W2 tanh(low), so that a step needs no kernel ahead of this one.
// That pays for a few sequences; with many, the eight CTAs of a head would each repeat the preparation ahead
// of their state arithmetic, and the preparation kernel runs first instead (PREPARED).
constexpr int STEP_MAX_RANK = 256;

template <typename T, typename TW, int R, bool PREPARED>
__global__ void __launch_bounds__(THREADS) delta_step_kernel(DeltaStateParams p) {
    __shared__ float rw_s[SLICES * R], au_s[SLICES * R], k_s[SLICES * R], w_s[SLICES * R];
    __shared__ float red[2][SLICES][COLS + 1];
    __shared__ float part[3][THREADS / 32];
    __shared__ float low_s[STEP_MAX_RANK];
    const int tid = threadIdx.x, jj = tid & (COLS - 1), g = tid >> 4;
    const int d = p.d, dv = p.dv;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int j = blockIdx.x * COLS + jj;
    const int64_t row = p.seq_q_start[seq];
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    float* S = p.state + (int64_t)slot * p.slot_stride + (int64_t)h * p.head_stride;
    const bool mine = j < dv;

    float st[R];
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int c = g + SLICES * i;
        st[i] = (mine && c < d) ? S[(int64_t)c * dv + j] : 0.f;
    }
    const T* rp = (const T*)p.rkv + row * p.row_stride;
    const float vj = mine ? to_f32<T>(rp[p.v_off + h * dv + j]) : 0.f;
    if (PREPARED) {
        for (int c = tid; c < SLICES * R; c += THREADS) {
            float rw = 0.f, au = 0.f, k = 0.f, w = 1.f;
            if (c < d) {
                w = p.decay[row * p.decay_stride + h * d + c];
                au = p.remove[row * p.remove_stride + h * d + c];
                k = to_f32<T>(rp[p.k_off + h * d + c]);
                rw = to_f32<T>(rp[p.r_off + h * d + c]) * w;
            }
            rw_s[c] = rw, au_s[c] = au, k_s[c] = k, w_s[c] = w;
        }
    }
    if (!PREPARED && p.low) {
        for (int i = tid; i < p.rank; i += THREADS) low_s[i] = tanhf(p.low[row * p.low_stride + i]);
        __syncthreads();
    }
    // the token's channels: up to two a thread
    float kv[2] = {0.f, 0.f}, rv[2] = {0.f, 0.f}, wv[2] = {1.f, 1.f}, av[2] = {0.f, 0.f};
    float kk = 0.f;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int c = tid + e * THREADS;
        if (!PREPARED && c < d && c < SLICES * R) {
            kv[e] = to_f32<T>(rp[p.k_off + h * d + c]);
            rv[e] = to_f32<T>(rp[p.r_off + h * d + c]);
            float z;
            if (p.low)
                z = dot_row<TW>((const TW*)p.w2 + (int64_t)(h * d + c) * p.rank, low_s, p.rank);
            else
                z = p.decay[row * p.decay_stride + h * d + c];
            wv[e] = expf(-p.decay_scale * sigmoid_f(z + (p.decay_bias ? p.decay_bias[h * d + c] : 0.f)));
            av[e] = sigmoid_f(p.remove[row * p.remove_stride + h * d + c] + (p.remove_bias ? p.remove_bias[h * d + c] : 0.f));
            kk = fmaf(kv[e], kv[e], kk);
        }
    }
    float inv, aur = 0.f, kr = 0.f;
    if (PREPARED) {
        const float4 t4 = *reinterpret_cast<const float4*>(p.dots + (row * p.heads + h) * 4);
        aur = t4.x, kr = t4.y, inv = t4.z;
        __syncthreads();
    } else {
    kk = warp_sum(kk);
    if ((tid & 31) == 0) part[0][tid >> 5] = kk;
    __syncthreads();
    inv = 1.0f / sqrtf(part[0][0] + part[0][1] + part[0][2] + part[0][3] + p.key_eps);
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int c = tid + e * THREADS;
        if (c < SLICES * R) {
            const float au = av[e] * (kv[e] * inv);
            rw_s[c] = rv[e] * wv[e], au_s[c] = au, k_s[c] = kv[e], w_s[c] = wv[e];
            aur = fmaf(au, rv[e], aur);
            kr = fmaf(kv[e], rv[e], kr);
        }
    }
    aur = warp_sum(aur);
    kr = warp_sum(kr);
    if ((tid & 31) == 0) part[1][tid >> 5] = aur, part[2][tid >> 5] = kr;
    __syncthreads();
    aur = part[1][0] + part[1][1] + part[1][2] + part[1][3];
    kr = part[2][0] + part[2][1] + part[2][2] + part[2][3];
    }
    float p1 = 0.f, p2 = 0.f;
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int c = g + SLICES * i;
        p1 = fmaf(k_s[c], st[i], p1);
        p2 = fmaf(rw_s[c], st[i], p2);
    }
    red[0][g][jj] = p1;
    red[1][g][jj] = p2;
    __syncthreads();
    p1 = p2 = 0.f;
#pragma unroll
    for (int s = 0; s < SLICES; s++) {
        p1 += red[0][s][jj];
        p2 += red[1][s][jj];
    }
    p1 *= inv;
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int c = g + SLICES * i;
        st[i] = fmaf(w_s[c], st[i], fmaf(k_s[c], vj, -au_s[c] * p1));
        if (mine && c < d) S[(int64_t)c * dv + j] = st[i];
    }
    if (g == 0 && mine) p.out[row * p.out_stride + h * dv + j] = p2 - aur * p1 + kr * vj;
}

template <typename T, int RC, int SL>
int launch_rc(const DeltaStateParams& p, cudaStream_t stream) {
    constexpr int P = (RC / 4) % 2 ? RC : RC + 4;
    constexpr int CL = 4 * (32 / SL);
    dim3 grid((p.dv + CL - 1) / CL, p.heads, p.nseq);
    const size_t smem = ((size_t)4 * TT * SL * P + 2 * TT * CL + 4 * TT + (size_t)SL * RC * (CL + 1)) * sizeof(float);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<T, RC, SL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) GB_REFUSE("delta_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    delta_scan_kernel<T, RC, SL><<<grid, THREADS, smem, stream>>>(p);
    GB_CHECK_LAUNCH("delta_scan");
    return 0;
}

template <typename T, typename TW, bool PREPARED>
int launch_step(const DeltaStateParams& p, dim3 grid, cudaStream_t stream) {
    if (p.d <= 64)
        delta_step_kernel<T, TW, 8, PREPARED><<<grid, THREADS, 0, stream>>>(p);
    else if (p.d <= 128)
        delta_step_kernel<T, TW, 16, PREPARED><<<grid, THREADS, 0, stream>>>(p);
    else
        delta_step_kernel<T, TW, 32, PREPARED><<<grid, THREADS, 0, stream>>>(p);
    GB_CHECK_LAUNCH("delta_step");
    return 0;
}

template <typename T>
int launch(const DeltaStateParams& p, int w2_dtype, cudaStream_t stream) {
    dim3 grid((p.dv + COLS - 1) / COLS, p.heads, p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("delta_scan: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    if (p.max_q_len == 1 && (p.low || !p.dots)) {      // every sequence brings one token and nothing is prepared: one kernel does it all
        if (p.low && w2_dtype == GB_BF16) return launch_step<T, __nv_bfloat16, false>(p, grid, stream);
        return launch_step<T, float, false>(p, grid, stream);
    }
    dim3 pgrid(p.rows, (p.heads + 3) / 4);
    if (pgrid.y > 65535) GB_REFUSE("delta_scan: %d heads exceed one launch", p.heads);
    delta_prep_kernel<T><<<pgrid, 128, 0, stream>>>(p);
    GB_CHECK_LAUNCH("delta_prep");
    if (p.max_q_len == 1) return launch_step<T, float, true>(p, grid, stream);
    const int rc = ((p.d + SLICES - 1) / SLICES + 3) / 4 * 4;
    switch (rc) {
        case 4: return launch_rc<T, 4, 8>(p, stream);
        case 8: return launch_rc<T, 8, 8>(p, stream);
        case 12: return launch_rc<T, 12, 8>(p, stream);
        case 16: return launch_rc<T, 16, 8>(p, stream);
        case 20: return launch_rc<T, 20, 8>(p, stream);
        case 24: return launch_rc<T, 24, 8>(p, stream);
        case 28: return launch_rc<T, 28, 8>(p, stream);
        case 32: return launch_rc<T, 32, 8>(p, stream);
    }
    GB_REFUSE("delta_scan: %d key channels a head; at most 256", p.d);
}

}  // namespace

GB_API int gb_delta_scan(const DeltaStateParams* pp, int dtype, int w2_dtype, cudaStream_t stream) {
    DeltaStateParams p = *pp;
    if (p.nseq <= 0 || p.rows <= 0) return 0;
    if (p.heads <= 0 || p.d <= 0 || p.d > 256 || p.dv <= 0) GB_REFUSE("delta_scan: %d heads of %d key and %d value channels", p.heads, p.d, p.dv);
    if (!p.rkv || !p.state || !p.out || !p.remove) GB_REFUSE("delta_scan: a tensor is missing");
    if (p.low) {
        if (p.max_q_len != 1 || !p.w2 || p.rank <= 0 || p.rank > STEP_MAX_RANK || (w2_dtype != GB_F32 && w2_dtype != GB_BF16))
            GB_REFUSE("delta_scan: the decay's second product is folded in only for single tokens and a rank up to %d (rank %d, rows of up to %d)",
                      STEP_MAX_RANK, p.rank, p.max_q_len);
    } else if (!p.decay) {
        GB_REFUSE("delta_scan: no decays");
    }
    if (p.max_q_len != 1 && !p.dots) GB_REFUSE("delta_scan: no room for the tokens' numbers");
    if (p.head_stride < (int64_t)p.d * p.dv || p.slot_stride < p.head_stride * p.heads) GB_REFUSE("delta_scan: the state is too small for its heads");
    if (dtype == GB_F32) return launch<float>(p, w2_dtype, stream);
    if (dtype == GB_BF16) return launch<__nv_bfloat16>(p, w2_dtype, stream);
    GB_REFUSE("delta_scan: unknown dtype %d", dtype);
}

GB_API int gb_delta_fused_max_rank() { return STEP_MAX_RANK; }

GB_API int gb_tanh(float* z, int rows, int cols, int64_t stride, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const int64_t n = (int64_t)rows * cols;
    tanh_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(z, rows, cols, stride);
    GB_CHECK_LAUNCH("tanh");
    return 0;
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_delta_state)
