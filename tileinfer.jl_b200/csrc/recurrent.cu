// Two recurrences whose only memory is a matrix state per (sequence, head), kept in 32-bit, and the small kernels around them.
//
//   decay scan (time mixing with a decay per key channel that depends on the token, and a bonus for the current token):
//       o_t = (S + diag(u) k_t v_t^T)^T r_t ;   S <- diag(w_t) S + k_t v_t^T ;   w_t = exp(-exp(d_t + w0))
//   delta scan (gated delta rule):
//       S <- g_t S ;  e = beta_t (v_t - S^T k_t) ;  S <- S + k_t e^T ;  o_t = S^T q_t
//       beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log) * softplus(a_t + dt_bias))
//
// S is [dim][vdim] (key rows, value columns). A block owns 32 value columns of one (sequence, head): lane = column, warp w owns
// the key rows 16 w .. 16 w + 15, sixteen state values per thread in registers. A step's tokens are walked in order from the
// state that earlier steps left, in batches of RS_BATCH tokens staged in shared memory (activations, decays and gates are
// computed while staging, in 32-bit); the partial sums of the warps are added in warp order, so a result depends on the
// token's place in its sequence alone, not on the batch or on how the prompt was cut.
#include "common.cuh"

#define RS_ROWS 16
#define RS_BATCH 16
#define RS_MAX_WARPS 16           // key sizes up to 256

__device__ __forceinline__ float rs_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float rs_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// The sequence of the step that token t belongs to: the last b with cu[b] <= t.
__device__ __forceinline__ int rs_sequence_of(const int* cu, int B, int t) {
    int lo = 0, hi = B - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldcg(cu + mid) <= t) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// ------------------------------------------------------------------------------------------------ decay scan
// rkv [n][ld] of T: r at r_off, k at k_off, v at v_off, heads of `D` side by side; dlog [n][H * D] float: the decay's logit
// before w0 [H * D] is added; u [H * D] float; state rows `state_stride` floats apart, a head's matrix at h * D * D.
// R key rows per thread (8 up to key size 128, so that a token's chain of dependent operations is short; 16 beyond). The next
// batch's rows are fetched into registers before this batch is worked on and laid into the other half of the staging buffers
// after it, so their latency hides behind the recurrence; one barrier per batch.
template <typename T, int R, int CB>
__global__ void decay_scan_kernel(float* __restrict__ o, const T* rkv, long long ld, int r_off, int k_off, int v_off, const float* dlog,
                                  const float* __restrict__ w0, const float* __restrict__ u, float* state, long long state_stride,
                                  const int* cu_seqlens, const int* seq_slots, int H, int D) {
    extern __shared__ __align__(16) float sm[];
    constexpr int SUBS = 32 / CB;                 // a warp's lanes: CB columns x SUBS groups of R rows
    constexpr int PER = RS_BATCH * R * SUBS / 32; // staged elements of r, k, w per thread and batch: RS_BATCH * Dp / threads
    constexpr int PV = (RS_BATCH * CB + 127) / 128;
    const int warps = blockDim.x >> 5, Dp = warps * R * SUBS, threads = blockDim.x;
    float* sr = sm;                               // [2][RS_BATCH][Dp]
    float* sk = sr + 2 * RS_BATCH * Dp;
    float* sw = sk + 2 * RS_BATCH * Dp;
    float* sv = sw + 2 * RS_BATCH * Dp;           // [2][RS_BATCH][CB]
    float* red = sv + 2 * RS_BATCH * CB;          // [2][RS_BATCH][warps][CB]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cl = lane % CB, sub = lane / CB;
    const int col0 = blockIdx.x * CB, col = col0 + cl, h = blockIdx.y, b = blockIdx.z;
    const int row0 = (warp * SUBS + sub) * R;
    const bool early_v = threads >= 128;          // enough threads to fetch a batch's values ahead in PV registers each
    pdl_enter();
    const int t0 = __ldcg(cu_seqlens + b), t1 = __ldcg(cu_seqlens + b + 1);
    float* S = state + (size_t)__ldcg(seq_slots + b) * state_stride + (size_t)h * D * D;
    float s[R], bonus[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const bool in = row0 + r < D && col < D;
        s[r] = in ? __ldcg(S + (size_t)(row0 + r) * D + col) : 0.f;
        bonus[r] = row0 + r < D ? u[h * D + row0 + r] : 0.f;
    }
    // Fetched values stay as they were loaded (no conversion, no branch): a use right behind a load would make the warp wait for it,
    // one round trip to memory per load instead of one per batch. Rows outside the batch or the head read a valid address and
    // are zeroed when they are laid into shared memory.
    T fr[PER], fk[PER], fv[PV];
    float fd[PER];
    auto fetch = [&](int base, int count) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = threadIdx.x + j * threads, i = e / Dp, d = e - i * Dp;
            const bool in = i < count && d < D;
            const size_t at = in ? (size_t)(base + i) * ld + h * D + d : 0;
            fr[j] = __ldcg(rkv + at + r_off);
            fk[j] = __ldcg(rkv + at + k_off);
            fd[j] = __ldcg(dlog + (in ? (size_t)(base + i) * H * D + h * D + d : 0));
        }
        if (early_v) {
#pragma unroll
            for (int j = 0; j < PV; ++j) {
                const int e = threadIdx.x + j * threads, i = e / CB, c = col0 + e % CB;
                const bool in = e < RS_BATCH * CB && i < count && c < D;
                fv[j] = __ldcg(rkv + (in ? (size_t)(base + i) * ld + v_off + h * D + c : 0));
            }
        }
    };
    auto stash = [&](int buf, int base, int count) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = threadIdx.x + j * threads, i = e / Dp, d = e - i * Dp;
            const bool in = i < count && d < D;
            sr[buf * RS_BATCH * Dp + e] = in ? to_f32(fr[j]) : 0.f;
            sk[buf * RS_BATCH * Dp + e] = in ? to_f32(fk[j]) : 0.f;
            sw[buf * RS_BATCH * Dp + e] = in ? expf(-expf(fd[j] + w0[h * D + d])) : 1.f;
        }
        if (early_v) {
#pragma unroll
            for (int j = 0; j < PV; ++j) {
                const int e = threadIdx.x + j * threads, i = e / CB, c = col0 + e % CB;
                if (e < RS_BATCH * CB) sv[buf * RS_BATCH * CB + e] = (i < count && c < D) ? to_f32(fv[j]) : 0.f;
            }
        } else {                                  // a block of few threads (a small key size) reads its values late
            for (int e = threadIdx.x; e < RS_BATCH * CB; e += threads) {
                const int i = e / CB, c = col0 + e % CB;
                sv[buf * RS_BATCH * CB + e] = (i < count && c < D) ? to_f32(__ldcg(rkv + (size_t)(base + i) * ld + v_off + h * D + c)) : 0.f;
            }
        }
    };
    if (t0 < t1) {
        fetch(t0, min(RS_BATCH, t1 - t0));
        stash(0, t0, min(RS_BATCH, t1 - t0));
    }
    __syncthreads();
    int it = 0;
    for (int base = t0; base < t1; base += RS_BATCH, ++it) {
        const int count = min(RS_BATCH, t1 - base), buf = it & 1;
        const int next = base + RS_BATCH, next_count = min(RS_BATCH, t1 - next);
        if (next < t1) fetch(next, next_count);
        float* my_red = red + (size_t)buf * RS_BATCH * warps * CB;
        for (int i = 0; i < count; ++i) {
            const float v = sv[(buf * RS_BATCH + i) * CB + cl];
            const float4* pr = reinterpret_cast<const float4*>(sr + (buf * RS_BATCH + i) * Dp + row0);
            const float4* pk = reinterpret_cast<const float4*>(sk + (buf * RS_BATCH + i) * Dp + row0);
            const float4* pw = reinterpret_cast<const float4*>(sw + (buf * RS_BATCH + i) * Dp + row0);
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int q = 0; q < R / 4; ++q) {
                const float4 r4 = pr[q], k4 = pk[q], w4 = pw[q];
                const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float kv = kk[c] * v;
                    part[c] = fmaf(fmaf(bonus[4 * q + c], kv, s[4 * q + c]), rr[c], part[c]);
                    s[4 * q + c] = fmaf(ww[c], s[4 * q + c], kv);
                }
            }
            float total = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
            for (int m = CB; m < 32; m <<= 1) total += __shfl_xor_sync(0xffffffffu, total, m);      // the row groups of a column
            if (sub == 0) my_red[(i * warps + warp) * CB + cl] = total;
        }
        if (next < t1) stash(buf ^ 1, next, next_count);
        __syncthreads();
        for (int e = threadIdx.x; e < count * CB; e += threads) {
            const int i = e / CB, c = col0 + e % CB;
            float total = 0.f;
            for (int w = 0; w < warps; ++w) total += my_red[(i * warps + w) * CB + e % CB];
            if (c < D) o[(size_t)(base + i) * H * D + h * D + c] = total;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
        if (row0 + r < D && col < D) S[(size_t)(row0 + r) * D + col] = s[r];
}

// One token per sequence (a decode step): no staging; a thread reads its rows' r, k and decay logits itself (the lanes of a warp
// read the same addresses), the warps' partial sums meet in a small array. The sums are added in the same order as in the scan.
template <typename T, int R>
__global__ void decay_token_kernel(float* __restrict__ o, const T* rkv, long long ld, int r_off, int k_off, int v_off, const float* dlog,
                                   const float* __restrict__ w0, const float* __restrict__ u, float* state, long long state_stride,
                                   const int* seq_slots, int H, int D) {
    __shared__ float red[RS_MAX_WARPS * 2 * 32];
    const int warps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane, h = blockIdx.y, t = blockIdx.z;
    const int row0 = warp * R;
    float* S = state + (size_t)__ldg(seq_slots + t) * state_stride + (size_t)h * D * D;
    float s[R], bonus[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {                 // the state does not depend on the step's other kernels: read before the wait
        s[r] = (row0 + r < D && col < D) ? __ldcg(S + (size_t)(row0 + r) * D + col) : 0.f;
        bonus[r] = row0 + r < D ? u[h * D + row0 + r] : 0.f;
    }
    pdl_enter();
    const T* row = rkv + (size_t)t * ld + h * D;
    const float v = col < D ? to_f32(__ldcg(row + v_off + col)) : 0.f;
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = row0 + r;
        float rr = 0.f, kk = 0.f, ww = 1.f;
        if (d < D) {
            rr = to_f32(__ldcg(row + r_off + d));
            kk = to_f32(__ldcg(row + k_off + d));
            ww = expf(-expf(__ldcg(dlog + (size_t)t * H * D + h * D + d) + w0[h * D + d]));
        }
        const float kv = kk * v;
        part[r & 3] = fmaf(fmaf(bonus[r], kv, s[r]), rr, part[r & 3]);
        s[r] = fmaf(ww, s[r], kv);
    }
    red[warp * 32 + lane] = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
    for (int r = 0; r < R; ++r)
        if (row0 + r < D && col < D) S[(size_t)(row0 + r) * D + col] = s[r];
    __syncthreads();
    if (warp == 0 && col < D) {
        float total = 0.f;
        for (int w = 0; w < warps; ++w) total += red[w * 32 + lane];
        o[(size_t)t * H * D + h * D + col] = total;
    }
}

template <typename T, int R, int CB>
static void launch_decay_scan(float* o, const T* rkv, long long ld, int r_off, int k_off, int v_off, const float* dlog, const float* w0, const float* u,
                              float* state, long long state_stride, const int* cu_seqlens, const int* seq_slots, int B, int H, int D, bool one_token,
                              cudaStream_t stream) {
    if (one_token) {
        ti_launch(decay_token_kernel<T, R>, dim3((D + 31) / 32, H, B), dim3((D + R - 1) / R * 32), 0, stream, o, rkv, ld, r_off, k_off, v_off, dlog, w0, u, state,
                  state_stride, seq_slots, H, D);
        return;
    }
    constexpr int RW = R * (32 / CB);             // key rows of a warp
    const int warps = (D + RW - 1) / RW;
    const size_t smem = (size_t)(2 * 3 * RS_BATCH * warps * RW + 2 * RS_BATCH * CB + 2 * RS_BATCH * warps * CB) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<T, R, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ti_launch(decay_scan_kernel<T, R, CB>, dim3((D + CB - 1) / CB, H, B), dim3(warps * 32), smem, stream, o, rkv, ld, r_off, k_off, v_off, dlog, w0, u, state,
              state_stride, cu_seqlens, seq_slots, H, D);
}

extern "C" int ti_decay_scan(float* o, const void* rkv, long long ld, int r_off, int k_off, int v_off, const float* dlog, const float* w0,
                             const float* u, float* state, long long state_stride, const int* cu_seqlens, const int* seq_slots, int n, int B,
                             int H, int D, int dtype, cudaStream_t stream) {
    if (n == 0 || B == 0) return 0;
    TI_REQUIRE(D > 0 && D <= RS_MAX_WARPS * RS_ROWS && H > 0, "decay_scan: %d heads of %d (at most %d)", H, D, RS_MAX_WARPS * RS_ROWS);
    // Very few (sequence, head) pairs: blocks of 16 or 8 columns, so that more SMs have one (the state's rows of a column are then
    // shared out among the lanes of a warp as well as among the warps). Every block stages all key rows of its head, so narrower
    // blocks multiply that work: with 64 blocks of 32 columns already (32 heads of 64, one prompt of 2,048 tokens) blocks of 16
    // columns were slower (551 against 465 us), hence only below a quarter of the SMs.
    const long long blocks32 = (long long)((D + 31) / 32) * H * B;
    const int sms = ti_sm_count();
#define RS_DECAY(R, CB) launch_decay_scan<T, R, CB>(o, (const T*)rkv, ld, r_off, k_off, v_off, dlog, w0, u, state, state_stride, cu_seqlens, seq_slots, B, H, D, n == B, stream)
    TI_DISPATCH_DTYPE(dtype, {
        if (D > 128) RS_DECAY(16, 32);
        else if (n == B || blocks32 * 4 >= sms) RS_DECAY(8, 32);
        else if (blocks32 * 8 >= sms) RS_DECAY(8, 16);
        else RS_DECAY(8, 8);
    });
#undef RS_DECAY
    return ti_check_launch("decay_scan");
}

// ------------------------------------------------------------------------------------------------ delta scan
// qkv [n][ld] float: q heads (G of D) at 0, k heads (G of D) at G * D, v heads (H of V) at 2 G D, already activated and
// normalised; ba [n][2 H] float: the logits of beta, then of the decay; head h reads q/k head h / (H / G). Sixteen key rows per
// thread; what a token reads out of the state before it writes (S^T k) is summed over the warps through shared memory, one barrier
// per token; the next batch's rows are fetched into registers while this batch is worked on.
template <int CB>
__global__ void delta_scan_kernel(float* __restrict__ o, const float* qkv, long long ld, const float* ba, const float* __restrict__ a_log,
                                  const float* __restrict__ dt_bias, float* state, long long state_stride, const int* cu_seqlens,
                                  const int* seq_slots, int H, int G, int D, int V) {
    extern __shared__ __align__(16) float sm[];
    constexpr int R = RS_ROWS, SUBS = 32 / CB;    // a warp's lanes: CB columns x SUBS groups of R rows
    constexpr int PER = RS_BATCH * R * SUBS / 32, PV = RS_BATCH * CB / 32;
    const int warps = blockDim.x >> 5, Dp = warps * R * SUBS, threads = blockDim.x;
    float* sq = sm;                               // [2][RS_BATCH][Dp]
    float* sk = sq + 2 * RS_BATCH * Dp;
    float* sv = sk + 2 * RS_BATCH * Dp;           // [2][RS_BATCH][CB]
    float* sg = sv + 2 * RS_BATCH * CB;           // [2][RS_BATCH][2]: decay, beta
    float* red = sg + 2 * RS_BATCH * 2;           // [2][warps][CB]
    float* red_o = red + 2 * warps * CB;          // [2][RS_BATCH][warps][CB]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cl = lane % CB, sub = lane / CB;
    const int col0 = blockIdx.x * CB, col = col0 + cl, h = blockIdx.y, b = blockIdx.z;
    const int g = h / (H / G), row0 = (warp * SUBS + sub) * R;
    pdl_enter();
    const int t0 = __ldcg(cu_seqlens + b), t1 = __ldcg(cu_seqlens + b + 1);
    float* S = state + (size_t)__ldcg(seq_slots + b) * state_stride + (size_t)h * D * V;
    const float rate = expf(a_log[h]), shift = dt_bias[h];
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = (row0 + r < D && col < V) ? __ldcg(S + (size_t)(row0 + r) * V + col) : 0.f;
    float fq[PER], fk[PER], fv[PV], fg[2];
    auto fetch = [&](int base, int count) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = threadIdx.x + j * threads, i = e / Dp, d = e - i * Dp;
            fq[j] = 0.f; fk[j] = 0.f;
            if (i < count && d < D) {
                const float* row = qkv + (size_t)(base + i) * ld + g * D + d;
                fq[j] = __ldcg(row);
                fk[j] = __ldcg(row + G * D);
            }
        }
#pragma unroll
        for (int j = 0; j < PV; ++j) {                // RS_BATCH * CB values over at least 32 threads
            const int e = threadIdx.x + j * threads, i = e / CB, c = col0 + e % CB;
            fv[j] = (e < RS_BATCH * CB && i < count && c < V) ? __ldcg(qkv + (size_t)(base + i) * ld + 2 * G * D + h * V + c) : 0.f;
        }
        if (threadIdx.x < count) {
            const float* row = ba + (size_t)(base + threadIdx.x) * 2 * H;
            fg[0] = __ldcg(row + H + h); fg[1] = __ldcg(row + h);
        }
    };
    auto stash = [&](int buf, int count) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = threadIdx.x + j * threads;
            sq[buf * RS_BATCH * Dp + e] = fq[j];
            sk[buf * RS_BATCH * Dp + e] = fk[j];
        }
#pragma unroll
        for (int j = 0; j < PV; ++j) {
            const int e = threadIdx.x + j * threads;
            if (e < RS_BATCH * CB) sv[buf * RS_BATCH * CB + e] = fv[j];
        }
        if (threadIdx.x < count) {
            sg[(buf * RS_BATCH + threadIdx.x) * 2] = expf(-rate * rs_softplus(fg[0] + shift));
            sg[(buf * RS_BATCH + threadIdx.x) * 2 + 1] = 1.0f / (1.0f + expf(-fg[1]));
        }
    };
    if (t0 < t1) {
        fetch(t0, min(RS_BATCH, t1 - t0));
        stash(0, min(RS_BATCH, t1 - t0));
    }
    __syncthreads();
    int it = 0, flip = 0;
    for (int base = t0; base < t1; base += RS_BATCH, ++it) {
        const int count = min(RS_BATCH, t1 - base), buf = it & 1;
        const int next = base + RS_BATCH, next_count = min(RS_BATCH, t1 - next);
        if (next < t1) fetch(next, next_count);
        float* my_red_o = red_o + (size_t)buf * RS_BATCH * warps * CB;
        for (int i = 0; i < count; ++i, flip ^= 1) {
            const float decay = sg[(buf * RS_BATCH + i) * 2], beta = sg[(buf * RS_BATCH + i) * 2 + 1];
            const float4* pq = reinterpret_cast<const float4*>(sq + (buf * RS_BATCH + i) * Dp + row0);
            const float4* pk = reinterpret_cast<const float4*>(sk + (buf * RS_BATCH + i) * Dp + row0);
            float kk[R];
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int q = 0; q < R / 4; ++q) {
                const float4 k4 = pk[q];
                kk[4 * q] = k4.x; kk[4 * q + 1] = k4.y; kk[4 * q + 2] = k4.z; kk[4 * q + 3] = k4.w;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    s[4 * q + c] *= decay;
                    part[c] = fmaf(s[4 * q + c], kk[4 * q + c], part[c]);
                }
            }
            float* buf_red = red + flip * warps * CB;
            float mine = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
            for (int m = CB; m < 32; m <<= 1) mine += __shfl_xor_sync(0xffffffffu, mine, m);        // the row groups of a column
            if (sub == 0) buf_red[warp * CB + cl] = mine;
            __syncthreads();
            float read = 0.f;
            for (int w = 0; w < warps; ++w) read += buf_red[w * CB + cl];         // every warp adds in the same order
            const float write = beta * (sv[(buf * RS_BATCH + i) * CB + cl] - read);
            float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int q = 0; q < R / 4; ++q) {
                const float4 q4 = pq[q];
                const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    s[4 * q + c] = fmaf(kk[4 * q + c], write, s[4 * q + c]);
                    out[c] = fmaf(s[4 * q + c], qq[c], out[c]);
                }
            }
            float mine_o = (out[0] + out[1]) + (out[2] + out[3]);
#pragma unroll
            for (int m = CB; m < 32; m <<= 1) mine_o += __shfl_xor_sync(0xffffffffu, mine_o, m);
            if (sub == 0) my_red_o[(i * warps + warp) * CB + cl] = mine_o;
        }
        if (next < t1) stash(buf ^ 1, next_count);
        __syncthreads();
        for (int e = threadIdx.x; e < count * CB; e += threads) {
            const int i = e / CB, c = col0 + e % CB;
            float total = 0.f;
            for (int w = 0; w < warps; ++w) total += my_red_o[(i * warps + w) * CB + e % CB];
            if (c < V) o[(size_t)(base + i) * H * V + h * V + c] = total;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
        if (row0 + r < D && col < V) S[(size_t)(row0 + r) * V + col] = s[r];
}

// One token per sequence: as the scan's step for one token, without staging.
__global__ void delta_token_kernel(float* __restrict__ o, const float* qkv, long long ld, const float* ba, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias, float* state, long long state_stride, const int* seq_slots, int H, int G,
                                   int D, int V) {
    constexpr int R = RS_ROWS;
    __shared__ float red[2 * RS_MAX_WARPS * 32];
    const int warps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane, h = blockIdx.y, t = blockIdx.z;
    const int g = h / (H / G), row0 = warp * R;
    float* S = state + (size_t)__ldg(seq_slots + t) * state_stride + (size_t)h * D * V;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = (row0 + r < D && col < V) ? __ldcg(S + (size_t)(row0 + r) * V + col) : 0.f;
    pdl_enter();
    const float* row = qkv + (size_t)t * ld;
    const float decay = expf(-expf(a_log[h]) * rs_softplus(__ldcg(ba + (size_t)t * 2 * H + H + h) + dt_bias[h]));
    const float beta = 1.0f / (1.0f + expf(-__ldcg(ba + (size_t)t * 2 * H + h)));
    const float v = col < V ? __ldcg(row + 2 * G * D + h * V + col) : 0.f;
    float kk[R], part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < R; ++r) {
        kk[r] = row0 + r < D ? __ldcg(row + G * D + g * D + row0 + r) : 0.f;
        s[r] *= decay;
        part[r & 3] = fmaf(s[r], kk[r], part[r & 3]);
    }
    red[warp * 32 + lane] = (part[0] + part[1]) + (part[2] + part[3]);
    __syncthreads();
    float read = 0.f;
    for (int w = 0; w < warps; ++w) read += red[w * 32 + lane];
    const float write = beta * (v - read);
    float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float qq = row0 + r < D ? __ldcg(row + g * D + row0 + r) : 0.f;
        s[r] = fmaf(kk[r], write, s[r]);
        out[r & 3] = fmaf(s[r], qq, out[r & 3]);
        if (row0 + r < D && col < V) S[(size_t)(row0 + r) * V + col] = s[r];
    }
    float* red_o = red + RS_MAX_WARPS * 32;
    red_o[warp * 32 + lane] = (out[0] + out[1]) + (out[2] + out[3]);
    __syncthreads();
    if (warp == 0 && col < V) {
        float total = 0.f;
        for (int w = 0; w < warps; ++w) total += red_o[w * 32 + lane];
        o[(size_t)t * H * V + h * V + col] = total;
    }
}

template <int CB>
static void launch_delta_scan(float* o, const float* qkv, long long ld, const float* ba, const float* a_log, const float* dt_bias, float* state,
                              long long state_stride, const int* cu_seqlens, const int* seq_slots, int B, int H, int G, int D, int V, cudaStream_t stream) {
    constexpr int RW = RS_ROWS * (32 / CB);       // key rows of a warp
    const int warps = (D + RW - 1) / RW;
    const size_t smem = (size_t)(2 * 2 * RS_BATCH * warps * RW + 2 * RS_BATCH * CB + 2 * RS_BATCH * 2 + 2 * warps * CB + 2 * RS_BATCH * warps * CB) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ti_launch(delta_scan_kernel<CB>, dim3((V + CB - 1) / CB, H, B), dim3(warps * 32), smem, stream, o, qkv, ld, ba, a_log, dt_bias, state, state_stride,
              cu_seqlens, seq_slots, H, G, D, V);
}

extern "C" int ti_delta_scan(float* o, const float* qkv, long long ld, const float* ba, const float* a_log, const float* dt_bias, float* state,
                             long long state_stride, const int* cu_seqlens, const int* seq_slots, int n, int B, int H, int G, int D, int V,
                             cudaStream_t stream) {
    if (n == 0 || B == 0) return 0;
    const int warps = (D + RS_ROWS - 1) / RS_ROWS;
    TI_REQUIRE(D > 0 && V > 0 && warps <= RS_MAX_WARPS, "delta_scan: keys of %d (at most %d)", D, RS_MAX_WARPS * RS_ROWS);
    TI_REQUIRE(H > 0 && G > 0 && H % G == 0, "delta_scan: %d heads do not divide into %d query/key heads", H, G);
    if (n == B) {                                 // one token per sequence
        ti_launch(delta_token_kernel, dim3((V + 31) / 32, H, B), dim3(warps * 32), 0, stream, o, qkv, ld, ba, a_log, dt_bias, state, state_stride, seq_slots,
                  H, G, D, V);
        return ti_check_launch("delta_token");
    }
    // Very few (sequence, head) pairs: blocks of 16 or 8 columns, so that more SMs have one and a token's barrier joins fewer warps
    // (with 64 blocks of 32 columns already, blocks of 16 were slower: 1,072 against 982 us; see the decay scan).
    const long long blocks32 = (long long)((V + 31) / 32) * H * B;
    const int sms = ti_sm_count();
    if (blocks32 * 4 >= sms) launch_delta_scan<32>(o, qkv, ld, ba, a_log, dt_bias, state, state_stride, cu_seqlens, seq_slots, B, H, G, D, V, stream);
    else if (blocks32 * 8 >= sms) launch_delta_scan<16>(o, qkv, ld, ba, a_log, dt_bias, state, state_stride, cu_seqlens, seq_slots, B, H, G, D, V, stream);
    else launch_delta_scan<8>(o, qkv, ld, ba, a_log, dt_bias, state, state_stride, cu_seqlens, seq_slots, B, H, G, D, V, stream);
    return ti_check_launch("delta_scan");
}

// ------------------------------------------------------------------------------------------------ blends with the token before
// out [K][n][W] of T (every blend a matrix of its own): out[k][t] = h_t + (h_(t-1) - h_t) * mu[k], h_(t-1) being the row before in the step, or for a sequence's
// first token of the step the row `prev` [slots] (state rows `prev_stride` floats apart; zeros at a sequence's start). The
// block of a sequence's first token then moves the state on to the sequence's last row of the step (it alone reads the state).
template <typename T>
__global__ void shift_blend_kernel(T* __restrict__ out, const T* h, const T* __restrict__ mu, int K, float* prev, long long prev_stride,
                                   const int* cu_seqlens, const int* seq_slots, int B, int W) {
    const int t = blockIdx.x;
    pdl_enter();
    const int b = rs_sequence_of(cu_seqlens, B, t);
    const int t0 = __ldcg(cu_seqlens + b), last = __ldcg(cu_seqlens + b + 1) - 1;
    float* st = prev + (size_t)__ldcg(seq_slots + b) * prev_stride;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float cur = to_f32(__ldcg(h + (size_t)t * W + c));
        const float before = t > t0 ? to_f32(__ldcg(h + (size_t)(t - 1) * W + c)) : __ldcg(st + c);
        for (int k = 0; k < K; ++k) out[((size_t)k * gridDim.x + t) * W + c] = from_f32<T>(fmaf(before - cur, to_f32(mu[(size_t)k * W + c]), cur));
        if (t == t0) st[c] = to_f32(__ldcg(h + (size_t)last * W + c));
    }
}

extern "C" int ti_shift_blend(void* out, const void* h, const void* mu, int K, float* prev, long long prev_stride, const int* cu_seqlens,
                              const int* seq_slots, int n, int B, int W, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(K > 0 && W > 0 && B > 0, "shift_blend: %d blends of rows of %d", K, W);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(shift_blend_kernel<T>, dim3(n), dim3(W >= 1024 ? 256 : 128), 0, stream, (T*)out, (const T*)h, (const T*)mu, K,
                                        prev, prev_stride, cu_seqlens, seq_slots, B, W)));
    return ti_check_launch("shift_blend");
}

// ------------------------------------------------------------------------------------------------ inputs of the delta scan
// proj [n][ld] of T: the projections' rows, C = 2 G D + H V channels (q heads, k heads, v heads). Every channel passes a causal
// convolution over time (conv [C][taps] of T, the last tap the current token's, zeros before the sequence's start; history from
// the step's own rows or from `hist`: the sequence's last taps - 1 rows, state rows `hist_stride` floats apart) and SiLU; then
// every q and k head becomes a unit vector x / sqrt(sum x^2 + unit_eps), q also times D^(-1/2). out [n][C] float.
#define DI_THREADS 256
template <typename T>
__global__ void __launch_bounds__(DI_THREADS) delta_inputs_kernel(float* __restrict__ out, const T* proj, long long ld, const T* __restrict__ conv,
                                                                   int taps, const float* hist, long long hist_stride, const int* cu_seqlens,
                                                                   const int* seq_slots, int B, int G, int D, int HV, float unit_eps) {
    extern __shared__ float y[];
    const int t = blockIdx.x, C = 2 * G * D + HV;
    pdl_enter();
    const int b = rs_sequence_of(cu_seqlens, B, t);
    const int t0 = __ldcg(cu_seqlens + b);
    const float* st = hist + (size_t)__ldcg(seq_slots + b) * hist_stride;
    for (int c = threadIdx.x; c < C; c += DI_THREADS) {
        float acc;
        if (taps <= 0) {
            acc = to_f32(__ldcg(proj + (size_t)t * ld + c));
        } else {
            acc = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int back = taps - 1 - j, tj = t - back;
                // Rows before the step's first of this sequence come from the state: its row taps - 1 - (t0 - tj) counts back from the newest.
                const float x = tj >= t0 ? to_f32(__ldcg(proj + (size_t)tj * ld + c)) : __ldcg(st + (size_t)(taps - 1 - (t0 - tj)) * C + c);
                acc = fmaf(to_f32(conv[(size_t)c * taps + j]), x, acc);
            }
        }
        y[c] = rs_silu(acc);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int hd = warp; hd < 2 * G; hd += DI_THREADS / 32) {              // a warp per q or k head
        float* src = y + (size_t)hd * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(src[d], src[d], ss);
        float inv = 1.0f / sqrtf(warp_sum(ss) + unit_eps);
        if (hd < G) inv *= 1.0f / sqrtf((float)D);
        for (int d = lane; d < D; d += 32) src[d] *= inv;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += DI_THREADS) out[(size_t)t * C + c] = y[c];
}

extern "C" int ti_delta_inputs(float* out, const void* proj, long long ld, const void* conv, int taps, const float* hist, long long hist_stride,
                               const int* cu_seqlens, const int* seq_slots, int n, int B, int G, int D, int HV, float unit_eps, int dtype,
                               cudaStream_t stream) {
    if (n == 0) return 0;
    const int C = 2 * G * D + HV;
    TI_REQUIRE(taps >= 0 && taps <= 64 && (taps <= 1 || hist != nullptr) && (taps == 0 || conv != nullptr), "delta_inputs: %d taps", taps);
    const size_t smem = (size_t)C * sizeof(float);
    TI_REQUIRE(smem <= 160 * 1024, "delta_inputs: %d channels", C);
    TI_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_inputs_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ti_launch(delta_inputs_kernel<T>, dim3(n), dim3(DI_THREADS), smem, stream, out, (const T*)proj, ld, (const T*)conv, taps, hist, hist_stride,
                  cu_seqlens, seq_slots, B, G, D, HV, unit_eps);
    });
    return ti_check_launch("delta_inputs");
}

// After the step: a sequence's history becomes its last taps - 1 projected rows (rows of this step where it brought enough, older
// ones moved up otherwise). A thread owns one channel of one sequence: it reads all it needs, then writes.
template <typename T>
__global__ void history_update_kernel(float* hist, long long hist_stride, const T* proj, long long ld, int taps, const int* cu_seqlens,
                                      const int* seq_slots, int C) {
    const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_enter();
    if (c >= C) return;
    const int t0 = __ldcg(cu_seqlens + b), t1 = __ldcg(cu_seqlens + b + 1), n = t1 - t0, keep = taps - 1;
    float* st = hist + (size_t)__ldcg(seq_slots + b) * hist_stride;
    float rows[64];
    for (int j = 0; j < keep; ++j) {
        const int back = keep - 1 - j;                       // row j of the new history lies `back` rows before the newest
        rows[j] = back < n ? to_f32(__ldcg(proj + (size_t)(t1 - 1 - back) * ld + c)) : __ldcg(st + (size_t)(j + n) * C + c);
    }
    for (int j = 0; j < keep; ++j) st[(size_t)j * C + c] = rows[j];
}

extern "C" int ti_history_update(float* hist, long long hist_stride, const void* proj, long long ld, int taps, const int* cu_seqlens,
                                 const int* seq_slots, int B, int C, int dtype, cudaStream_t stream) {
    if (B == 0 || taps <= 1) return 0;
    TI_REQUIRE(taps <= 64, "history_update: %d taps", taps);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(history_update_kernel<T>, dim3((C + 127) / 128, B), dim3(128), 0, stream, hist, hist_stride, (const T*)proj,
                                        ld, taps, cu_seqlens, seq_slots, C)));
    return ti_check_launch("history_update");
}

// ------------------------------------------------------------------------------------------------ a scan's output
// y [n][H * V] of T = o / rms(o over a head) * w * silu(gate): every head normed by itself in 32-bit; w is [V] (one weight for all
// heads, `shared_w`) or [H * V]; gate [n][ldg] of T holds the gate's projection. A warp per (token, head).
template <typename T>
__global__ void heads_norm_gate_kernel(T* __restrict__ y, const float* o, const T* gate, long long ldg, const T* __restrict__ w, int shared_w,
                                       float eps, int H, int V, size_t heads_total) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= heads_total) return;
    const size_t t = item / H;
    const int h = (int)(item % H);
    const float* src = o + (t * H + h) * V;
    float ss = 0.f;
    for (int d = lane; d < V; d += 32) {
        const float v = __ldcg(src + d);
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)V + eps);
    for (int d = lane; d < V; d += 32) {
        float v = __ldcg(src + d) * inv * to_f32(w[shared_w ? d : h * V + d]);
        if (gate != nullptr) v *= rs_silu(to_f32(__ldcg(gate + t * ldg + h * V + d)));
        y[(t * H + h) * V + d] = from_f32<T>(v);
    }
}

extern "C" int ti_heads_norm_gate(void* y, const float* o, const void* gate, long long ldg, const void* w, int shared_w, float eps, int n, int H,
                                  int V, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    const size_t total = (size_t)n * H;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(heads_norm_gate_kernel<T>, dim3((unsigned)((total + 3) / 4)), dim3(128), 0, stream, (T*)y, o, (const T*)gate,
                                        ldg, (const T*)w, shared_w, eps, H, V, total)));
    return ti_check_launch("heads_norm_gate");
}

// ------------------------------------------------------------------------------------------------ two mixers side by side
// out [n][size] float = sa * A' + sb * B'; A' = A / rms(A over the row) * wa with `normed`, else A (the same for B). A and B are rows
// of T or the sum of 32-bit partial sums (a product cut over k). One block per token.
template <typename T>
__device__ __forceinline__ float pair_value(const T* d, const float* partials, int n_partials, size_t stride, size_t at) {
    if (partials != nullptr) {
        float v = __ldcg(partials + at);
        for (int s = 1; s < n_partials; ++s) v += __ldcg(partials + (size_t)s * stride + at);
        return v;
    }
    return to_f32(__ldcg(d + at));
}

template <typename T>
__global__ void pair_combine_kernel(float* __restrict__ out, const T* a, const float* pa, int na, size_t sa_stride, const T* b, const float* pb,
                                    int nb, size_t sb_stride, const T* __restrict__ wa, const T* __restrict__ wb, int normed, float eps,
                                    float scale_a, float scale_b, int size) {
    extern __shared__ float rows[];                // [2][size]
    __shared__ float scratch[33];
    pdl_enter();
    float ssa = 0.f, ssb = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const size_t at = (size_t)blockIdx.x * size + i;
        const float va = pair_value<T>(a, pa, na, sa_stride, at), vb = pair_value<T>(b, pb, nb, sb_stride, at);
        rows[i] = va; rows[size + i] = vb;
        ssa = fmaf(va, va, ssa); ssb = fmaf(vb, vb, ssb);
    }
    float ia = 1.f, ib = 1.f;
    if (normed) {
        ia = 1.0f / sqrtf(block_sum(ssa, scratch) / (float)size + eps);
        ib = 1.0f / sqrtf(block_sum(ssb, scratch) / (float)size + eps);
    }
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float va = rows[i], vb = rows[size + i];
        if (normed) { va = va * ia * to_f32(wa[i]); vb = vb * ib * to_f32(wb[i]); }
        out[(size_t)blockIdx.x * size + i] = fmaf(scale_a, va, scale_b * vb);
    }
}

extern "C" int ti_pair_combine(float* out, const void* a, const float* pa, int na, long long sa_stride, const void* b, const float* pb, int nb,
                               long long sb_stride, const void* wa, const void* wb, int normed, float eps, float scale_a, float scale_b, int n,
                               int size, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(!normed || (wa != nullptr && wb != nullptr), "pair_combine: normed outputs need their weights");
    const size_t smem = (size_t)2 * size * sizeof(float);
    TI_REQUIRE(smem <= 160 * 1024, "pair_combine: rows of %d", size);
    TI_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(pair_combine_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ti_launch(pair_combine_kernel<T>, dim3(n), dim3(size >= 1024 ? 256 : 128), smem, stream, out, (const T*)a, pa, na, (size_t)sa_stride, (const T*)b,
                  pb, nb, (size_t)sb_stride, (const T*)wa, (const T*)wb, normed, eps, scale_a, scale_b, size);
    });
    return ti_check_launch("pair_combine");
}
