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
template <typename T>
__global__ void decay_scan_kernel(float* __restrict__ o, const T* rkv, long long ld, int r_off, int k_off, int v_off, const float* dlog,
                                  const float* __restrict__ w0, const float* __restrict__ u, float* state, long long state_stride,
                                  const int* cu_seqlens, const int* seq_slots, int H, int D) {
    extern __shared__ float sm[];
    const int warps = blockDim.x >> 5, Dp = warps * RS_ROWS;
    float* sr = sm;                               // [RS_BATCH][Dp]
    float* sk = sr + RS_BATCH * Dp;
    float* sw = sk + RS_BATCH * Dp;
    float* sv = sw + RS_BATCH * Dp;               // [RS_BATCH][32]
    float* red = sv + RS_BATCH * 32;              // [RS_BATCH][warps][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane, h = blockIdx.y, b = blockIdx.z;
    const int row0 = warp * RS_ROWS;
    pdl_enter();
    const int t0 = __ldcg(cu_seqlens + b), t1 = __ldcg(cu_seqlens + b + 1);
    float* S = state + (size_t)__ldcg(seq_slots + b) * state_stride + (size_t)h * D * D;
    float s[RS_ROWS], bonus[RS_ROWS];
#pragma unroll
    for (int r = 0; r < RS_ROWS; ++r) {
        const bool in = row0 + r < D && col < D;
        s[r] = in ? __ldcg(S + (size_t)(row0 + r) * D + col) : 0.f;
        bonus[r] = row0 + r < D ? u[h * D + row0 + r] : 0.f;
    }
    for (int base = t0; base < t1; base += RS_BATCH) {
        const int count = min(RS_BATCH, t1 - base);
        __syncthreads();                                   // the batch before has been read
        for (int e = threadIdx.x; e < count * Dp; e += blockDim.x) {
            const int i = e / Dp, d = e % Dp;
            float rr = 0.f, kk = 0.f, ww = 1.f;
            if (d < D) {
                const T* row = rkv + (size_t)(base + i) * ld + h * D + d;
                rr = to_f32(__ldcg(row + r_off));
                kk = to_f32(__ldcg(row + k_off));
                ww = expf(-expf(__ldcg(dlog + (size_t)(base + i) * H * D + h * D + d) + w0[h * D + d]));
            }
            sr[e] = rr; sk[e] = kk; sw[e] = ww;
        }
        for (int e = threadIdx.x; e < count * 32; e += blockDim.x) {
            const int i = e >> 5, c = blockIdx.x * 32 + (e & 31);
            sv[e] = c < D ? to_f32(__ldcg(rkv + (size_t)(base + i) * ld + v_off + h * D + c)) : 0.f;
        }
        __syncthreads();
        for (int i = 0; i < count; ++i) {
            const float v = sv[i * 32 + lane];
            const float* pr = sr + i * Dp + row0;
            const float* pk = sk + i * Dp + row0;
            const float* pw = sw + i * Dp + row0;
            float part = 0.f;
#pragma unroll
            for (int r = 0; r < RS_ROWS; ++r) {
                const float kv = pk[r] * v;
                part = fmaf(fmaf(bonus[r], kv, s[r]), pr[r], part);
                s[r] = fmaf(pw[r], s[r], kv);
            }
            red[(i * warps + warp) * 32 + lane] = part;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < count * 32; e += blockDim.x) {
            const int i = e >> 5, c = blockIdx.x * 32 + (e & 31);
            float total = 0.f;
            for (int w = 0; w < warps; ++w) total += red[(i * warps + w) * 32 + (e & 31)];
            if (c < D) o[(size_t)(base + i) * H * D + h * D + c] = total;
        }
    }
#pragma unroll
    for (int r = 0; r < RS_ROWS; ++r)
        if (row0 + r < D && col < D) S[(size_t)(row0 + r) * D + col] = s[r];
}

extern "C" int ti_decay_scan(float* o, const void* rkv, long long ld, int r_off, int k_off, int v_off, const float* dlog, const float* w0,
                             const float* u, float* state, long long state_stride, const int* cu_seqlens, const int* seq_slots, int n, int B,
                             int H, int D, int dtype, cudaStream_t stream) {
    if (n == 0 || B == 0) return 0;
    const int warps = (D + RS_ROWS - 1) / RS_ROWS;
    TI_REQUIRE(D > 0 && warps <= RS_MAX_WARPS && H > 0, "decay_scan: %d heads of %d (at most %d)", H, D, RS_MAX_WARPS * RS_ROWS);
    const size_t smem = (size_t)(3 * RS_BATCH * warps * RS_ROWS + RS_BATCH * 32 + RS_BATCH * warps * 32) * sizeof(float);
    dim3 grid((D + 31) / 32, H, B);
    TI_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ti_launch(decay_scan_kernel<T>, grid, dim3(warps * 32), smem, stream, o, (const T*)rkv, ld, r_off, k_off, v_off, dlog, w0, u, state,
                  state_stride, cu_seqlens, seq_slots, H, D);
    });
    return ti_check_launch("decay_scan");
}

// ------------------------------------------------------------------------------------------------ delta scan
// qkv [n][ld] float: q heads (G of D) at 0, k heads (G of D) at G * D, v heads (H of V) at 2 G D, already activated and
// normalised; ba [n][2 H] float: the logits of beta, then of the decay; head h reads q/k head h / (H / G).
__global__ void delta_scan_kernel(float* __restrict__ o, const float* qkv, long long ld, const float* ba, const float* __restrict__ a_log,
                                  const float* __restrict__ dt_bias, float* state, long long state_stride, const int* cu_seqlens,
                                  const int* seq_slots, int H, int G, int D, int V) {
    extern __shared__ float sm[];
    const int warps = blockDim.x >> 5, Dp = warps * RS_ROWS;
    float* sq = sm;                               // [RS_BATCH][Dp]
    float* sk = sq + RS_BATCH * Dp;
    float* sv = sk + RS_BATCH * Dp;               // [RS_BATCH][32]
    float* sg = sv + RS_BATCH * 32;               // [RS_BATCH][2]: decay, beta
    float* red = sg + RS_BATCH * 2;               // [2][warps][32]
    float* red_o = red + 2 * warps * 32;          // [RS_BATCH][warps][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane, h = blockIdx.y, b = blockIdx.z;
    const int g = h / (H / G), row0 = warp * RS_ROWS;
    pdl_enter();
    const int t0 = __ldcg(cu_seqlens + b), t1 = __ldcg(cu_seqlens + b + 1);
    float* S = state + (size_t)__ldcg(seq_slots + b) * state_stride + (size_t)h * D * V;
    const float rate = expf(a_log[h]), shift = dt_bias[h];
    float s[RS_ROWS];
#pragma unroll
    for (int r = 0; r < RS_ROWS; ++r) s[r] = (row0 + r < D && col < V) ? __ldcg(S + (size_t)(row0 + r) * V + col) : 0.f;
    for (int base = t0; base < t1; base += RS_BATCH) {
        const int count = min(RS_BATCH, t1 - base);
        __syncthreads();
        for (int e = threadIdx.x; e < count * Dp; e += blockDim.x) {
            const int i = e / Dp, d = e % Dp;
            const float* row = qkv + (size_t)(base + i) * ld + g * D + d;
            sq[e] = d < D ? __ldcg(row) : 0.f;
            sk[e] = d < D ? __ldcg(row + G * D) : 0.f;
        }
        for (int e = threadIdx.x; e < count * 32; e += blockDim.x) {
            const int i = e >> 5, c = blockIdx.x * 32 + (e & 31);
            sv[e] = c < V ? __ldcg(qkv + (size_t)(base + i) * ld + 2 * G * D + h * V + c) : 0.f;
        }
        for (int i = threadIdx.x; i < count; i += blockDim.x) {
            const float* row = ba + (size_t)(base + i) * 2 * H;
            sg[2 * i] = expf(-rate * rs_softplus(__ldcg(row + H + h) + shift));
            sg[2 * i + 1] = 1.0f / (1.0f + expf(-__ldcg(row + h)));
        }
        __syncthreads();
        for (int i = 0; i < count; ++i) {
            const float decay = sg[2 * i], beta = sg[2 * i + 1];
            const float* pq = sq + i * Dp + row0;
            const float* pk = sk + i * Dp + row0;
            float part = 0.f;
#pragma unroll
            for (int r = 0; r < RS_ROWS; ++r) {
                s[r] *= decay;
                part = fmaf(s[r], pk[r], part);
            }
            float* buf = red + (i & 1) * warps * 32;
            buf[warp * 32 + lane] = part;
            __syncthreads();
            float read = 0.f;
            for (int w = 0; w < warps; ++w) read += buf[w * 32 + lane];       // every warp adds in the same order
            const float write = beta * (sv[i * 32 + lane] - read);
            float out = 0.f;
#pragma unroll
            for (int r = 0; r < RS_ROWS; ++r) {
                s[r] = fmaf(pk[r], write, s[r]);
                out = fmaf(s[r], pq[r], out);
            }
            red_o[(i * warps + warp) * 32 + lane] = out;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < count * 32; e += blockDim.x) {
            const int i = e >> 5, c = blockIdx.x * 32 + (e & 31);
            float total = 0.f;
            for (int w = 0; w < warps; ++w) total += red_o[(i * warps + w) * 32 + (e & 31)];
            if (c < V) o[(size_t)(base + i) * H * V + h * V + c] = total;
        }
    }
#pragma unroll
    for (int r = 0; r < RS_ROWS; ++r)
        if (row0 + r < D && col < V) S[(size_t)(row0 + r) * V + col] = s[r];
}

extern "C" int ti_delta_scan(float* o, const float* qkv, long long ld, const float* ba, const float* a_log, const float* dt_bias, float* state,
                             long long state_stride, const int* cu_seqlens, const int* seq_slots, int n, int B, int H, int G, int D, int V,
                             cudaStream_t stream) {
    if (n == 0 || B == 0) return 0;
    const int warps = (D + RS_ROWS - 1) / RS_ROWS;
    TI_REQUIRE(D > 0 && V > 0 && warps <= RS_MAX_WARPS, "delta_scan: keys of %d (at most %d)", D, RS_MAX_WARPS * RS_ROWS);
    TI_REQUIRE(H > 0 && G > 0 && H % G == 0, "delta_scan: %d heads do not divide into %d query/key heads", H, G);
    const size_t smem = (size_t)(2 * RS_BATCH * warps * RS_ROWS + RS_BATCH * 32 + RS_BATCH * 2 + 2 * warps * 32 + RS_BATCH * warps * 32) * sizeof(float);
    dim3 grid((V + 31) / 32, H, B);
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ti_launch(delta_scan_kernel, grid, dim3(warps * 32), smem, stream, o, qkv, ld, ba, a_log, dt_bias, state, state_stride, cu_seqlens, seq_slots,
              H, G, D, V);
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
