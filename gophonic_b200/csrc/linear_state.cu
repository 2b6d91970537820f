// Mixers that carry a matrix state per head instead of keys and values: for every token
//
//     S <- diag(a_t) S + b_t k_t v_t^T          (S is d x dv, fp32, one per sequence and head)
//     o_t = S^T q_t
//
// with a_t a decay per key channel (gated linear attention) or one number per head (the matrix
// memory of an mLSTM, where b_t is the input gate and a further column n <- a_t n + b_t k_t gives
// the normaliser).  State, decays, gates and the sums are fp32 whatever the activation dtype;
// q, k and v are read as the projection left them.
//
// The recurrence runs token by token, in order, for prompts and single tokens alike, so the state
// after a token is the same bits however the sequence was cut into steps and whatever else the
// batch holds.  Work is spread over (sequence, head, block of 16 value columns): columns of S are
// independent of one another.  Inside a CTA a warp owns 4 columns and its 8 groups of lanes own a
// slice of the key channels each; a thread keeps its d/8 state elements in registers across all
// tokens of the step, the tokens' q, k and decay rows are staged in shared memory eight tokens at a
// time, and a token's output is a shuffle sum over the 8 slices.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace {

constexpr int COLS = 16;     // value columns per CTA
constexpr int SLICES = 8;    // slices of the key channels
constexpr int TT = 8;        // tokens staged at a time
constexpr int THREADS = 128;
static_assert(TT * COLS == THREADS, "a thread fetches one value of a tile");
static_assert(TT == SLICES, "the exchange that adds the slices up leaves one token's sum with each slice");

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------------------------------------
// decay of gated linear attention, in place: z[r, c] <- sigmoid(z[r, c] + bias[c]) ^ (1 / tau)
__global__ void gla_decay_kernel(float* __restrict__ z, const float* __restrict__ bias, int64_t total, int width, float inv_tau) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float x = z[i] + (bias ? bias[i % width] : 0.f);
    z[i] = expf(log_sigmoid(x) * inv_tau);
}

// ------------------------------------------------------------------------------------------
// gates of the matrix memory.  One warp per (sequence, head), 32 tokens at a time: the lanes take a
// token each for the capped gates, the running maximum m_t = max(f_t + m_(t-1), i_t) is walked in
// order through shuffles (an add and a max a token), then the lanes turn their token's values into
// the factors keep_t = exp(f_t + m_(t-1) - m_t) and take_t = exp(i_t - m_t).
// coef[r, h] = (keep, take, m_t, -): the last place is filled by the scan's normaliser column.
__global__ void __launch_bounds__(32) mlstm_gates_kernel(LinearStateParams p) {
    const int h = blockIdx.x, seq = blockIdx.y, lane = threadIdx.x;
    const int q_len = p.seq_q_len[seq], q_start = p.seq_q_start[seq];
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    float* m_state = p.state + (int64_t)slot * p.slot_stride + (int64_t)h * p.head_stride + (int64_t)p.d * p.dv + p.d;
    float m = *m_state;
    const float cap = p.gate_cap, inv_cap = 1.f / p.gate_cap;
    const float bi = p.gate_bias ? p.gate_bias[h] : 0.f, bf = p.gate_bias ? p.gate_bias[p.heads + h] : 0.f;
    for (int t0 = 0; t0 < q_len; t0 += 32) {
        const int t = t0 + lane;
        float gi = 0.f, gf = 0.f;
        if (t < q_len) {
            const float* g = p.gates + (int64_t)(q_start + t) * p.gates_stride;
            gi = cap * tanhf((g[h] + bi) * inv_cap);
            gf = log_sigmoid(cap * tanhf((g[p.heads + h] + bf) * inv_cap));
        }
        float m_before = 0.f, m_mine = 0.f;
        const int n = q_len - t0 < 32 ? q_len - t0 : 32;
        for (int j = 0; j < n; j++) {
            const float fj = __shfl_sync(0xffffffffu, gf, j), ij = __shfl_sync(0xffffffffu, gi, j);
            const float m_new = fmaxf(fj + m, ij);
            if (lane == j) {
                m_before = m;
                m_mine = m_new;
            }
            m = m_new;
        }
        if (t < q_len) {
            float4 c;
            c.x = expf(gf + m_before - m_mine);
            c.y = expf(gi - m_mine);
            c.z = m_mine;
            c.w = 1.f;
            *reinterpret_cast<float4*>(p.coef + ((int64_t)(q_start + t) * p.heads + h) * 4) = c;
        }
    }
    if (lane == 0) *m_state = m;
}

// ------------------------------------------------------------------------------------------
// the scan.  RC: key channels per slice (a multiple of 4, RC * 8 >= d).  SCALAR: one decay per head
// and token (coef), with the input gate folded into the staged keys and one more block of columns
// for the normaliser; otherwise a decay per key channel (p.decay).
template <typename T, int RC, bool SCALAR>
__global__ void __launch_bounds__(THREADS) state_scan_kernel(LinearStateParams p) {
    constexpr int P = (RC / 4) % 2 ? RC : RC + 4;   // slice stride in floats: P / 4 odd, so the 8 slices' 16-byte reads miss each other's banks
    constexpr int ROW = SLICES * P;
    __shared__ __align__(16) float q_s[TT][ROW];
    __shared__ __align__(16) float k_s[TT][ROW];
    __shared__ __align__(16) float a_s[SCALAR ? 1 : TT][SCALAR ? 4 : ROW];
    __shared__ float v_s[TT][COLS];
    __shared__ float o_s[TT][COLS];
    __shared__ float keep_s[TT], m_s[TT];
    __shared__ float st_s[SLICES * RC][COLS + 1];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slice = lane & 7, col = warp * 4 + (lane >> 3);   // this thread's slice and column of the CTA's 16
    const int d = p.d, dv = p.dv, H = p.heads;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int vblocks = (dv + COLS - 1) / COLS;
    const bool norm_col = SCALAR && (int)blockIdx.x == vblocks;   // the block that carries n instead of columns of S
    const int j0 = blockIdx.x * COLS;
    const int q_len = p.seq_q_len[seq], q_start = p.seq_q_start[seq];
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    float* S = p.state + (int64_t)slot * p.slot_stride + (int64_t)h * p.head_stride;
    float* nvec = S + (int64_t)d * dv;

    // the state block of this CTA, through shared memory so that global rows are read whole: 16 bytes a
    // thread where the block's rows are whole and aligned
    const bool vec = !norm_col && !(dv & 3) && j0 + COLS <= dv && !((uintptr_t)(S + j0) & 15);
    if (vec) {
#pragma unroll 4
        for (int idx = tid; idx < SLICES * RC * (COLS / 4); idx += THREADS) {
            const int c = idx / (COLS / 4), q4 = idx % (COLS / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < d) v = *reinterpret_cast<const float4*>(S + (int64_t)c * dv + j0 + 4 * q4);
            st_s[c][4 * q4] = v.x;
            st_s[c][4 * q4 + 1] = v.y;
            st_s[c][4 * q4 + 2] = v.z;
            st_s[c][4 * q4 + 3] = v.w;
        }
    }
    for (int idx = tid; !vec && idx < SLICES * RC * COLS; idx += THREADS) {
        const int c = idx / COLS, jj = idx % COLS;
        float v = 0.f;
        if (c < d) {
            if (norm_col)
                v = jj == 0 ? nvec[c] : 0.f;
            else if (j0 + jj < dv)
                v = S[(int64_t)c * dv + j0 + jj];
        }
        st_s[c][jj] = v;
    }
    __syncthreads();
    float st[RC];
#pragma unroll
    for (int i = 0; i < RC; i++) st[i] = st_s[slice * RC + i][col];

    const T* base = (const T*)p.qkv;
    // A tile's rows are fetched into registers while the tile before it is worked on, and put into
    // shared memory between two barriers: the global loads' latency hides behind the arithmetic.
    constexpr int PER = TT * SLICES * RC / THREADS;   // q/k/decay elements a thread fetches per tile
    // Every load of a fetch is unconditional (indices clamped into the tile) and nothing is done with the
    // values until they are stored: they are all in flight at once.  What lies outside the tile or the
    // head is replaced when it is stored: a token or channel that is not there changes nothing (decay 1, key 0).
    T rq[PER], rk[PER], rv;
    float ra[PER], rkeep = 1.f, rm = 0.f;
    auto fetch = [&](int t0) {
        const int nt = q_len - t0 < TT ? q_len - t0 : TT;
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = tid + e * THREADS;
            int t = idx / (SLICES * RC), c = idx % (SLICES * RC);
            t = t < nt ? t : nt - 1;
            c = c < d ? c : d - 1;
            const int64_t row = q_start + t0 + t;
            const T* r = base + row * p.row_stride;
            rq[e] = r[p.q_off + h * d + c];
            rk[e] = r[p.k_off + h * d + c];
            ra[e] = SCALAR ? p.coef[(row * H + h) * 4 + 1] : p.decay[row * p.decay_stride + h * d + c];
        }
        {
            int t = tid / COLS, jj = j0 + tid % COLS;      // TT * COLS == THREADS
            t = t < nt ? t : nt - 1;
            jj = jj < dv ? jj : dv - 1;
            rv = base[(int64_t)(q_start + t0 + t) * p.row_stride + p.v_off + h * dv + jj];
        }
        if (SCALAR) {
            const int64_t row = q_start + t0 + (tid < nt ? tid : nt - 1);
            rkeep = p.coef[(row * H + h) * 4];
            rm = p.coef[(row * H + h) * 4 + 2];
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
            const int at = (c / RC) * P + c % RC;
            const bool there = t < nt && c < d;
            q_s[t][at] = there ? to_f32<T>(rq[e]) * p.q_scale : 0.f;
            // one decay per head: the input gate goes into the key, the decay itself is keep_s
            k_s[t][at] = there ? (SCALAR ? to_f32<T>(rk[e]) * ra[e] : to_f32<T>(rk[e])) : 0.f;
            if (!SCALAR) a_s[t][at] = there ? ra[e] : 1.f;
        }
        {
            const int t = tid / COLS, jj = tid % COLS;
            float v = 0.f;
            if (t < nt) {
                if (norm_col)
                    v = jj == 0 ? 1.f : 0.f;
                else if (j0 + jj < dv)
                    v = to_f32<T>(rv);
            }
            v_s[t][jj] = v;
        }
        if (SCALAR && tid < TT) {
            keep_s[tid] = tid < nt ? rkeep : 1.f;
            m_s[tid] = rm;
        }
        __syncthreads();
        if (t0 + TT < q_len) fetch(t0 + TT);
        // All eight tokens of the tile, unrolled (a tile's missing tokens leave the state as it is: decay 1,
        // key 0).  A thread's sums over its slice of the channels stay in registers until the tile is done;
        // then three exchange steps add the eight slices up and leave token t's sum with the lane of slice t.
        float acc[TT];
#pragma unroll
        for (int t = 0; t < TT; t++) {
            const float vj = v_s[t][col];
            const float keep = SCALAR ? keep_s[t] : 0.f;
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
            for (int i = 0; i < RC; i += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(&q_s[t][slice * P + i]);
                const float4 k4 = *reinterpret_cast<const float4*>(&k_s[t][slice * P + i]);
                float4 a4 = make_float4(keep, keep, keep, keep);
                if (!SCALAR) a4 = *reinterpret_cast<const float4*>(&a_s[t][slice * P + i]);
                st[i] = fmaf(a4.x, st[i], k4.x * vj);
                st[i + 1] = fmaf(a4.y, st[i + 1], k4.y * vj);
                st[i + 2] = fmaf(a4.z, st[i + 2], k4.z * vj);
                st[i + 3] = fmaf(a4.w, st[i + 3], k4.w * vj);
                acc0 = fmaf(st[i], q4.x, acc0);
                acc1 = fmaf(st[i + 1], q4.y, acc1);
                acc2 = fmaf(st[i + 2], q4.z, acc2);
                acc3 = fmaf(st[i + 3], q4.w, acc3);
            }
            acc[t] = (acc0 + acc1) + (acc2 + acc3);
        }
        float b4[4], b2[2], total;
        {
            const bool up = slice & 4;
#pragma unroll
            for (int j = 0; j < 4; j++) b4[j] = (up ? acc[j + 4] : acc[j]) + __shfl_xor_sync(0xffffffffu, up ? acc[j] : acc[j + 4], 4);
        }
        {
            const bool up = slice & 2;
#pragma unroll
            for (int j = 0; j < 2; j++) b2[j] = (up ? b4[j + 2] : b4[j]) + __shfl_xor_sync(0xffffffffu, up ? b4[j] : b4[j + 2], 2);
        }
        {
            const bool up = slice & 1;
            total = (up ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, up ? b2[0] : b2[1], 1);
        }
        o_s[slice][col] = total;
        __syncthreads();
        if (norm_col) {
            // n . q of the tile's tokens -> the divisor max(|n . q|, exp(-m)) + 1e-6
            if (tid < nt) {
                const int64_t row = q_start + t0 + tid;
                p.coef[(row * H + h) * 4 + 3] = fmaxf(fabsf(o_s[tid][0]), expf(-m_s[tid])) + 1e-6f;
            }
        } else {
            for (int idx = tid; idx < nt * COLS; idx += THREADS) {
                const int t = idx / COLS, jj = idx % COLS;
                if (j0 + jj < dv) p.out[(int64_t)(q_start + t0 + t) * p.out_stride + h * dv + j0 + jj] = o_s[t][jj];
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RC; i++) st_s[slice * RC + i][col] = st[i];
    __syncthreads();
    if (vec) {
#pragma unroll 4
        for (int idx = tid; idx < SLICES * RC * (COLS / 4); idx += THREADS) {
            const int c = idx / (COLS / 4), q4 = idx % (COLS / 4);
            if (c < d)
                *reinterpret_cast<float4*>(S + (int64_t)c * dv + j0 + 4 * q4) =
                    make_float4(st_s[c][4 * q4], st_s[c][4 * q4 + 1], st_s[c][4 * q4 + 2], st_s[c][4 * q4 + 3]);
        }
    }
    for (int idx = tid; !vec && idx < SLICES * RC * COLS; idx += THREADS) {
        const int c = idx / COLS, jj = idx % COLS;
        if (c >= d) continue;
        if (norm_col) {
            if (jj == 0) nvec[c] = st_s[c][0];
        } else if (j0 + jj < dv) {
            S[(int64_t)c * dv + j0 + jj] = st_s[c][jj];
        }
    }
}

// ------------------------------------------------------------------------------------------
// The same scan for heads of 128 or 256 key channels, laid out so that shared memory is read once: a
// warp owns 4 columns and its 32 lanes are 32 slices of the channels (RC = d / 32 each), a thread keeps
// RC x 4 state elements.  A token's q, k and decay rows are then read by the warp as whole rows (every
// lane its own 16 bytes, no two quarter-warps the same bytes), four times less shared-memory traffic
// than with 8 slices and a column a thread, for the same registers.  A tile's 8 tokens x 4 columns of
// sums are added up over the 32 slices by a five-step exchange that leaves each lane one of them.
template <typename T, int RC, bool SCALAR>
__global__ void __launch_bounds__(THREADS) state_scan_wide_kernel(LinearStateParams p) {
    constexpr int D = 32 * RC;          // key channels of a head
    constexpr int CW = 4;               // columns a warp (and a thread) owns
    __shared__ __align__(16) float q_s[TT][D];
    __shared__ __align__(16) float k_s[TT][D];
    __shared__ __align__(16) float a_s[SCALAR ? 1 : TT][SCALAR ? 4 : D];
    __shared__ __align__(16) float v_s[TT][COLS];
    __shared__ float o_s[TT][COLS];
    __shared__ float keep_s[TT], m_s[TT];
    __shared__ float st_s[D][COLS + 1];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int dv = p.dv, H = p.heads;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int vblocks = (dv + COLS - 1) / COLS;
    const bool norm_col = SCALAR && (int)blockIdx.x == vblocks;
    const int j0 = blockIdx.x * COLS;
    const int q_len = p.seq_q_len[seq], q_start = p.seq_q_start[seq];
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    float* S = p.state + (int64_t)slot * p.slot_stride + (int64_t)h * p.head_stride;
    float* nvec = S + (int64_t)D * dv;

    const bool vec = !norm_col && !(dv & 3) && j0 + COLS <= dv && !((uintptr_t)(S + j0) & 15);
    if (vec) {
#pragma unroll 4
        for (int idx = tid; idx < D * (COLS / 4); idx += THREADS) {
            const int c = idx / (COLS / 4), q4 = idx % (COLS / 4);
            const float4 v = *reinterpret_cast<const float4*>(S + (int64_t)c * dv + j0 + 4 * q4);
            st_s[c][4 * q4] = v.x;
            st_s[c][4 * q4 + 1] = v.y;
            st_s[c][4 * q4 + 2] = v.z;
            st_s[c][4 * q4 + 3] = v.w;
        }
    }
    for (int idx = tid; !vec && idx < D * COLS; idx += THREADS) {
        const int c = idx / COLS, jj = idx % COLS;
        float v = 0.f;
        if (norm_col)
            v = jj == 0 ? nvec[c] : 0.f;
        else if (j0 + jj < dv)
            v = S[(int64_t)c * dv + j0 + jj];
        st_s[c][jj] = v;
    }
    __syncthreads();
    float st[RC][CW];
#pragma unroll
    for (int i = 0; i < RC; i++)
#pragma unroll
        for (int c = 0; c < CW; c++) st[i][c] = st_s[lane * RC + i][warp * CW + c];

    const T* base = (const T*)p.qkv;
    constexpr int PER = TT * D / THREADS;
    T rq[PER], rk[PER], rv;
    float ra[PER], rkeep = 1.f, rm = 0.f;
    auto fetch = [&](int t0) {
        const int nt = q_len - t0 < TT ? q_len - t0 : TT;
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = tid + e * THREADS;
            int t = idx / D;
            const int c = idx % D;
            t = t < nt ? t : nt - 1;
            const int64_t row = q_start + t0 + t;
            const T* r = base + row * p.row_stride;
            rq[e] = r[p.q_off + h * D + c];
            rk[e] = r[p.k_off + h * D + c];
            ra[e] = SCALAR ? p.coef[(row * H + h) * 4 + 1] : p.decay[row * p.decay_stride + h * D + c];
        }
        {
            int t = tid / COLS, jj = j0 + tid % COLS;
            t = t < nt ? t : nt - 1;
            jj = jj < dv ? jj : dv - 1;
            rv = base[(int64_t)(q_start + t0 + t) * p.row_stride + p.v_off + h * dv + jj];
        }
        if (SCALAR) {
            const int64_t row = q_start + t0 + (tid < nt ? tid : nt - 1);
            rkeep = p.coef[(row * H + h) * 4];
            rm = p.coef[(row * H + h) * 4 + 2];
        }
    };
    if (q_len > 0) fetch(0);
    for (int t0 = 0; t0 < q_len; t0 += TT) {
        const int nt = q_len - t0 < TT ? q_len - t0 : TT;
        __syncthreads();
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = tid + e * THREADS;
            const int t = idx / D, c = idx % D;
            const bool there = t < nt;
            q_s[t][c] = there ? to_f32<T>(rq[e]) * p.q_scale : 0.f;
            k_s[t][c] = there ? (SCALAR ? to_f32<T>(rk[e]) * ra[e] : to_f32<T>(rk[e])) : 0.f;
            if (!SCALAR) a_s[t][c] = there ? ra[e] : 1.f;
        }
        {
            const int t = tid / COLS, jj = tid % COLS;
            float v = 0.f;
            if (t < nt) {
                if (norm_col)
                    v = jj == 0 ? 1.f : 0.f;
                else if (j0 + jj < dv)
                    v = to_f32<T>(rv);
            }
            v_s[t][jj] = v;
        }
        if (SCALAR && tid < TT) {
            keep_s[tid] = tid < nt ? rkeep : 1.f;
            m_s[tid] = rm;
        }
        __syncthreads();
        if (t0 + TT < q_len) fetch(t0 + TT);
        float acc[TT * CW];     // index t * 4 + c
#pragma unroll
        for (int t = 0; t < TT; t++) {
            const float4 v4 = *reinterpret_cast<const float4*>(&v_s[t][warp * CW]);
            const float vv[CW] = {v4.x, v4.y, v4.z, v4.w};
            const float keep = SCALAR ? keep_s[t] : 0.f;
            float sum[CW] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < RC; i += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(&q_s[t][lane * RC + i]);
                const float4 k4 = *reinterpret_cast<const float4*>(&k_s[t][lane * RC + i]);
                float4 a4 = make_float4(keep, keep, keep, keep);
                if (!SCALAR) a4 = *reinterpret_cast<const float4*>(&a_s[t][lane * RC + i]);
                const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int u = 0; u < 4; u++)
#pragma unroll
                    for (int c = 0; c < CW; c++) {
                        st[i + u][c] = fmaf(aa[u], st[i + u][c], kk[u] * vv[c]);
                        sum[c] = fmaf(st[i + u][c], qq[u], sum[c]);
                    }
            }
#pragma unroll
            for (int c = 0; c < CW; c++) acc[t * CW + c] = sum[c];
        }
        // 32 sums a thread over 32 slices: halve the sums and the lanes five times
        float b16[16], b8[8], b4[4], b2[2], total;
        {
            const bool up = lane & 16;
#pragma unroll
            for (int j = 0; j < 16; j++) b16[j] = (up ? acc[j + 16] : acc[j]) + __shfl_xor_sync(0xffffffffu, up ? acc[j] : acc[j + 16], 16);
        }
        {
            const bool up = lane & 8;
#pragma unroll
            for (int j = 0; j < 8; j++) b8[j] = (up ? b16[j + 8] : b16[j]) + __shfl_xor_sync(0xffffffffu, up ? b16[j] : b16[j + 8], 8);
        }
        {
            const bool up = lane & 4;
#pragma unroll
            for (int j = 0; j < 4; j++) b4[j] = (up ? b8[j + 4] : b8[j]) + __shfl_xor_sync(0xffffffffu, up ? b8[j] : b8[j + 4], 4);
        }
        {
            const bool up = lane & 2;
#pragma unroll
            for (int j = 0; j < 2; j++) b2[j] = (up ? b4[j + 2] : b4[j]) + __shfl_xor_sync(0xffffffffu, up ? b4[j] : b4[j + 2], 2);
        }
        {
            const bool up = lane & 1;
            total = (up ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, up ? b2[0] : b2[1], 1);
        }
        o_s[lane >> 2][warp * CW + (lane & 3)] = total;     // lane l is left with sum number l = t * 4 + c
        __syncthreads();
        if (norm_col) {
            if (tid < nt) {
                const int64_t row = q_start + t0 + tid;
                p.coef[(row * H + h) * 4 + 3] = fmaxf(fabsf(o_s[tid][0]), expf(-m_s[tid])) + 1e-6f;
            }
        } else {
            for (int idx = tid; idx < nt * COLS; idx += THREADS) {
                const int t = idx / COLS, jj = idx % COLS;
                if (j0 + jj < dv) p.out[(int64_t)(q_start + t0 + t) * p.out_stride + h * dv + j0 + jj] = o_s[t][jj];
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RC; i++)
#pragma unroll
        for (int c = 0; c < CW; c++) st_s[lane * RC + i][warp * CW + c] = st[i][c];
    __syncthreads();
    if (vec) {
#pragma unroll 4
        for (int idx = tid; idx < D * (COLS / 4); idx += THREADS) {
            const int c = idx / (COLS / 4), q4 = idx % (COLS / 4);
            *reinterpret_cast<float4*>(S + (int64_t)c * dv + j0 + 4 * q4) =
                make_float4(st_s[c][4 * q4], st_s[c][4 * q4 + 1], st_s[c][4 * q4 + 2], st_s[c][4 * q4 + 3]);
        }
    }
    for (int idx = tid; !vec && idx < D * COLS; idx += THREADS) {
        const int c = idx / COLS, jj = idx % COLS;
        if (norm_col) {
            if (jj == 0) nvec[c] = st_s[c][0];
        } else if (j0 + jj < dv) {
            S[(int64_t)c * dv + j0 + jj] = st_s[c][jj];
        }
    }
}

// ------------------------------------------------------------------------------------------
// One token for every sequence (a decode step): the work is reading and writing the state once.  A CTA
// owns 16 columns of one head's S; thread (group g of 8, column j of 16) takes the channels g, g + 8, ...
// so that a warp's loads are whole 64-byte rows, keeps them in registers from load to store, and the
// eight groups' sums meet in shared memory.  All state loads are issued before anything waits.
template <typename T, int R, bool SCALAR>
__global__ void __launch_bounds__(THREADS) state_step_kernel(LinearStateParams p) {
    __shared__ float q_s[SLICES * R], k_s[SLICES * R], a_s[SLICES * R];
    __shared__ float red[SLICES][COLS + 1];
    const int tid = threadIdx.x, jj = tid & (COLS - 1), g = tid >> 4;
    const int d = p.d, dv = p.dv, H = p.heads;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int vblocks = (dv + COLS - 1) / COLS;
    const bool norm_col = SCALAR && (int)blockIdx.x == vblocks;
    const int j = blockIdx.x * COLS + jj;
    const int64_t row = p.seq_q_start[seq];
    int slot = p.seq_slot[seq];
    if (!gb_check(slot, p.max_slots, GB_CHECK_SLOT)) slot = 0;
    float* S = p.state + (int64_t)slot * p.slot_stride + (int64_t)h * p.head_stride;
    float* nvec = S + (int64_t)d * dv;
    const bool mine = norm_col ? jj == 0 : j < dv;

    float st[R];
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int c = g + SLICES * i;
        st[i] = (mine && c < d) ? (norm_col ? nvec[c] : S[(int64_t)c * dv + j]) : 0.f;
    }
    const T* r = (const T*)p.qkv + row * p.row_stride;
    float keep = 0.f, take = 1.f, m = 0.f;
    if (SCALAR) {
        const float* cf = p.coef + (row * H + h) * 4;
        keep = cf[0];
        take = cf[1];
        m = cf[2];
    }
    for (int c = tid; c < SLICES * R; c += THREADS) {
        const bool there = c < d;
        q_s[c] = there ? to_f32<T>(r[p.q_off + h * d + c]) * p.q_scale : 0.f;
        k_s[c] = there ? to_f32<T>(r[p.k_off + h * d + c]) * take : 0.f;
        a_s[c] = SCALAR ? keep : (there ? p.decay[row * p.decay_stride + h * d + c] : 1.f);
    }
    const float vj = norm_col ? 1.f : (j < dv ? to_f32<T>(r[p.v_off + h * dv + j]) : 0.f);
    __syncthreads();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int c = g + SLICES * i;
        st[i] = fmaf(a_s[c], st[i], k_s[c] * vj);
        acc = fmaf(st[i], q_s[c], acc);
    }
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int c = g + SLICES * i;
        if (mine && c < d) {
            if (norm_col)
                nvec[c] = st[i];
            else
                S[(int64_t)c * dv + j] = st[i];
        }
    }
    red[g][jj] = acc;
    __syncthreads();
    if (tid < COLS) {
        float total = 0.f;
#pragma unroll
        for (int s = 0; s < SLICES; s++) total += red[s][tid];
        if (norm_col) {
            if (tid == 0) p.coef[(row * H + h) * 4 + 3] = fmaxf(fabsf(total), expf(-m)) + 1e-6f;
        } else if (j < dv) {
            p.out[row * p.out_stride + h * dv + j] = total;
        }
    }
}

template <typename T, bool SCALAR>
int launch_step(const LinearStateParams& p, cudaStream_t stream) {
    dim3 grid((p.dv + COLS - 1) / COLS + (SCALAR ? 1 : 0), p.heads, p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("state_scan: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    if (p.d <= 64)
        state_step_kernel<T, 8, SCALAR><<<grid, THREADS, 0, stream>>>(p);
    else if (p.d <= 128)
        state_step_kernel<T, 16, SCALAR><<<grid, THREADS, 0, stream>>>(p);
    else
        state_step_kernel<T, 32, SCALAR><<<grid, THREADS, 0, stream>>>(p);
    GB_CHECK_LAUNCH("state_step");
    return 0;
}

template <typename T, bool SCALAR>
int launch_scan(const LinearStateParams& p, cudaStream_t stream) {
    if (p.max_q_len == 1) return launch_step<T, SCALAR>(p, stream);   // every sequence brings one token
    const int rc = ((p.d + SLICES - 1) / SLICES + 3) / 4 * 4;
    dim3 grid((p.dv + COLS - 1) / COLS + (SCALAR ? 1 : 0), p.heads, p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("state_scan: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    if (p.d == 128 || p.d == 256) {     // heads whose channels fill a warp's 32 slices: shared memory read once
        if (p.d == 128)
            state_scan_wide_kernel<T, 4, SCALAR><<<grid, THREADS, 0, stream>>>(p);
        else
            state_scan_wide_kernel<T, 8, SCALAR><<<grid, THREADS, 0, stream>>>(p);
        GB_CHECK_LAUNCH("state_scan");
        return 0;
    }
    switch (rc) {
        case 4: state_scan_kernel<T, 4, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        case 8: state_scan_kernel<T, 8, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        case 12: state_scan_kernel<T, 12, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        case 16: state_scan_kernel<T, 16, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        case 20: state_scan_kernel<T, 20, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        case 24: state_scan_kernel<T, 24, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        case 28: state_scan_kernel<T, 28, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        case 32: state_scan_kernel<T, 32, SCALAR><<<grid, THREADS, 0, stream>>>(p); break;
        default: GB_REFUSE("state_scan: %d key channels a head; at most 256", p.d);
    }
    GB_CHECK_LAUNCH("state_scan");
    return 0;
}

int check(const LinearStateParams& p, const char* who) {
    if (p.heads <= 0 || p.d <= 0 || p.d > 256 || p.dv <= 0) GB_REFUSE("%s: %d heads of %d key and %d value channels", who, p.heads, p.d, p.dv);
    if (!p.qkv || !p.state || !p.out) GB_REFUSE("%s: a tensor is missing", who);
    if (p.head_stride < (int64_t)p.d * p.dv || p.slot_stride < p.head_stride * p.heads) GB_REFUSE("%s: the state is too small for its heads", who);
    return 0;
}

// ------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void load4(const T* p, float* out);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x, out[1] = v.y, out[2] = v.z, out[3] = v.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float* out) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x), b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    out[0] = __low2float(a), out[1] = __high2float(a), out[2] = __low2float(b), out[3] = __high2float(b);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float* in);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float* in) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float* in) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(in[0], in[1]), b = __floats2bfloat162_rn(in[2], in[3]);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&a);
    v.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = v;
}

// per (row, head): y = norm(x / div) * w * gate(g), everything optional but the gate.  One warp a head.
template <typename TI, typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(HeadGateParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = blockIdx.x;
    const int h = blockIdx.y * 4 + warp;
    if (h >= p.heads) return;
    const int n = p.size;
    const TI* x = (const TI*)p.x + r * p.x_stride + (int64_t)h * n;
    const T* g = (const T*)p.gate + r * p.gate_stride + (int64_t)h * n;
    T* y = (T*)p.y + r * p.y_stride + (int64_t)h * n;
    const float div = p.divisor ? p.divisor[(r * p.heads + h) * p.divisor_stride] : 1.f;
    const float* w = p.weight ? p.weight + (p.weight_per_head ? (int64_t)h * n : 0) : nullptr;
    // heads of up to 256: every lane keeps its elements in registers, so x is read once and all of a
    // lane's loads (x, gate, weight) are in flight together
    if (n <= 256) {
        float v[8], z[8], ww[8];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int i = lane + 32 * e;
            const bool in = i < n;
            v[e] = in ? to_f32<TI>(x[i]) : 0.f;
            z[e] = in ? to_f32<T>(g[i]) : 0.f;
            ww[e] = (in && w) ? w[i] : 1.f;
        }
#pragma unroll
        for (int e = 0; e < 8; e++) {
            if (p.divisor) v[e] /= div;
            ss += v[e] * v[e];
        }
        float inv = 1.f;
        if (p.normed) inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + p.eps);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int i = lane + 32 * e;
            if (i >= n) continue;
            float o = v[e];
            if (p.normed) o *= inv;
            if (w) o *= ww[e];
            const float sg = 1.f / (1.f + expf(-z[e]));
            o *= p.gate_kind == 1 ? z[e] * sg : sg;
            y[i] = from_f32<T>(o);
        }
        return;
    }
    float ss = 0.f;
    if (p.normed) {
        for (int i = lane; i < n; i += 32) {
            const float v = to_f32<TI>(x[i]) / div;
            ss += v * v;
        }
        ss = warp_sum(ss);
    }
    const float inv = p.normed ? 1.0f / sqrtf(ss / (float)n + p.eps) : 1.f;
    for (int i = lane; i < n; i += 32) {
        float v = to_f32<TI>(x[i]);
        if (p.divisor) v /= div;
        if (p.normed) v *= inv;
        if (w) v *= w[i];
        const float z = to_f32<T>(g[i]);
        const float s = 1.f / (1.f + expf(-z));
        v *= p.gate_kind == 1 ? z * s : s;
        y[i] = from_f32<T>(v);
    }
}

// The same for heads of 128, 256, 384 or 512 whose rows are aligned.  A warp takes a span of up to 512
// neighbouring elements of a row, which is 4, 2 or 1 whole heads (HB); a lane takes four neighbouring
// elements of each 128 as one load (16 bytes of float32, 8 of bfloat16), all of them issued before
// anything is computed: a head of 128 alone is too few bytes in flight a warp to keep the memory busy.
template <typename TI, typename T>
__global__ void __launch_bounds__(128) head_norm_gate_span_kernel(HeadGateParams p, int hb) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = blockIdx.x;
    const int h0 = (blockIdx.y * 4 + warp) * hb;
    if (h0 >= p.heads) return;
    const int n = p.size, nv = n >> 7;                 // 128-element chunks a head
    const int heads_here = p.heads - h0 < hb ? p.heads - h0 : hb;
    const int chunks = heads_here * nv;                // <= 4
    const TI* x = (const TI*)p.x + r * p.x_stride + (int64_t)h0 * n;
    const T* g = (const T*)p.gate + r * p.gate_stride + (int64_t)h0 * n;
    T* y = (T*)p.y + r * p.y_stride + (int64_t)h0 * n;
    float v[16], z[16], ww[16], dv4[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        dv4[e] = 1.f;
        if (e < chunks) {
            const int i = 128 * e + 4 * lane;
            load4<TI>(x + i, v + 4 * e);
            load4<T>(g + i, z + 4 * e);
            if (p.weight) {
                const float* w = p.weight + (p.weight_per_head ? (int64_t)h0 * n + i : i % n);
                const float4 w4 = *reinterpret_cast<const float4*>(w);
                ww[4 * e] = w4.x, ww[4 * e + 1] = w4.y, ww[4 * e + 2] = w4.z, ww[4 * e + 3] = w4.w;
            }
            if (p.divisor) dv4[e] = p.divisor[(r * p.heads + h0 + e / nv) * p.divisor_stride];
        }
    }
    float ss[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        ss[e] = 0.f;
        if (e < chunks) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (p.divisor) v[4 * e + u] /= dv4[e];
                ss[e] += v[4 * e + u] * v[4 * e + u];
            }
        }
    }
    float inv[4] = {1.f, 1.f, 1.f, 1.f};
    if (p.normed) {
#pragma unroll
        for (int e = 0; e < 4; e++) ss[e] = warp_sum(ss[e]);
        // a head's sum of squares: its chunks' sums, in order
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (e < chunks) {
                const int first = (e / nv) * nv;
                float t = 0.f;
#pragma unroll
                for (int f = 0; f < 4; f++)
                    if (f >= first && f < first + nv) t += ss[f];
                inv[e] = 1.0f / sqrtf(t / (float)n + p.eps);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < 4; e++) {
        if (e < chunks) {
            float o[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float t = v[4 * e + u];
                if (p.normed) t *= inv[e];
                if (p.weight) t *= ww[4 * e + u];
                const float zz = z[4 * e + u];
                const float sg = 1.f / (1.f + expf(-zz));
                o[u] = t * (p.gate_kind == 1 ? zz * sg : sg);
            }
            store4<T>(y + 128 * e + 4 * lane, o);
        }
    }
}

template <typename TI, typename T>
int launch_gate(const HeadGateParams& p, cudaStream_t stream) {
    const int n = p.size;
    const bool aligned = !((uintptr_t)p.x & (4 * sizeof(TI) - 1)) && !(p.x_stride & 3) && !((uintptr_t)p.gate & (4 * sizeof(T) - 1)) &&
                         !(p.gate_stride & 3) && !((uintptr_t)p.y & (4 * sizeof(T) - 1)) && !(p.y_stride & 3) && !((uintptr_t)p.weight & 15);
    if (!(n & 127) && n <= 512 && aligned) {
        const int hb = 512 / n;     // whole heads in a span of 512 elements
        dim3 grid(p.rows, (p.heads + 4 * hb - 1) / (4 * hb));
        if (grid.y > 65535) GB_REFUSE("head_norm_gate: %d heads exceed one launch", p.heads);
        head_norm_gate_span_kernel<TI, T><<<grid, 128, 0, stream>>>(p, hb);
        GB_CHECK_LAUNCH("head_norm_gate");
        return 0;
    }
    dim3 grid(p.rows, (p.heads + 3) / 4);
    if (grid.y > 65535) GB_REFUSE("head_norm_gate: %d heads exceed one launch", p.heads);
    head_norm_gate_kernel<TI, T><<<grid, 128, 0, stream>>>(p);
    GB_CHECK_LAUNCH("head_norm_gate");
    return 0;
}

}  // namespace

GB_API int gb_gla_decay(float* z, const float* bias, int rows, int width, float tau, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || !(tau > 0.f)) GB_REFUSE("gla_decay: width %d, tau %g", width, (double)tau);
    const int64_t total = (int64_t)rows * width;
    gla_decay_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(z, bias, total, width, 1.f / tau);
    GB_CHECK_LAUNCH("gla_decay");
    return 0;
}

GB_API int gb_state_scan(const LinearStateParams* pp, int dtype, cudaStream_t stream) {
    LinearStateParams p = *pp;
    if (p.nseq <= 0) return 0;
    if (int rc = check(p, "state_scan")) return rc;
    if (p.scalar_decay) {
        if (!p.coef || !p.gates || !(p.gate_cap > 0.f)) GB_REFUSE("state_scan: gates, their cap (%g) or room for the factors is missing", (double)p.gate_cap);
        if (p.head_stride < (int64_t)p.d * p.dv + p.d + 1) GB_REFUSE("state_scan: the state has no room for the normaliser and the maximum");
        mlstm_gates_kernel<<<dim3(p.heads, p.nseq), 32, 0, stream>>>(p);
        GB_CHECK_LAUNCH("mlstm_gates");
        if (dtype == GB_F32) return launch_scan<float, true>(p, stream);
        if (dtype == GB_BF16) return launch_scan<__nv_bfloat16, true>(p, stream);
    } else {
        if (!p.decay) GB_REFUSE("state_scan: no decays");
        if (dtype == GB_F32) return launch_scan<float, false>(p, stream);
        if (dtype == GB_BF16) return launch_scan<__nv_bfloat16, false>(p, stream);
    }
    GB_REFUSE("state_scan: unknown dtype %d", dtype);
}

GB_API int gb_head_norm_gate(const HeadGateParams* pp, int x_dtype, int dtype, cudaStream_t stream) {
    HeadGateParams p = *pp;
    if (p.rows <= 0) return 0;
    if (p.heads <= 0 || p.size <= 0) GB_REFUSE("head_norm_gate: %d heads of %d", p.heads, p.size);
    if (p.gate_kind != 0 && p.gate_kind != 1) GB_REFUSE("head_norm_gate: gate kind %d", p.gate_kind);
    if (dtype == GB_F32 && x_dtype == GB_F32) return launch_gate<float, float>(p, stream);
    if (dtype == GB_BF16 && x_dtype == GB_F32) return launch_gate<float, __nv_bfloat16>(p, stream);
    if (dtype == GB_BF16 && x_dtype == GB_BF16) return launch_gate<__nv_bfloat16, __nv_bfloat16>(p, stream);
    GB_REFUSE("head_norm_gate: input dtype %d with output dtype %d", x_dtype, dtype);
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_linear_state)
