// The inputs of an attention layer whose projections pass through a short causal convolution over time:
//
//   u_t = T(W h_t + b)                                    the projection's row (the product comes rounded to T; the bias is added here)
//   y_t[c] = T( sum_j conv[c][j] * u_(t - taps + 1 + j)[c] )   zeros before the sequence's start
//   q, k  <- y / rms(y over the WHOLE row of q, or of k) * w    (weights as long as the row; optional)
//            or, with head_norm, every head by itself: y_h / rms(y_h) * w, one weight of the head's size for all heads
//   q, k  <- rotation of the first `rotary` elements of every head by the position's angles (optional)
//   q -> q_out [n, heads, Dp]; k, v -> their place in the paged cache [pages][kv_heads][page][Dp]
//
// Dp >= the query/key size and the value size: rows are filled up with zeros, which changes neither a score nor an output.
// The last taps - 1 rows u of every sequence are its convolution state [slots][taps - 1][channels] (32-bit copies of the
// T values, so a row read from the state equals the row read from the step's own projection bit for bit); tokens at the
// start of a step read it, and `conv_state_update` (a second launch: the first one's blocks read what it overwrites)
// moves it on. One block per token; everything between the loads and the one rounding per stage is 32-bit.
#include "common.cuh"

#define CI_THREADS 256
#define CI_MAX_TAPS 16

// The sequence of the step that token t belongs to: the last b with cu[b] <= t.
__device__ __forceinline__ int sequence_of(const int* cu, int B, int t) {
    int lo = 0, hi = B - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldcg(cu + mid) <= t) lo = mid; else hi = mid - 1;
    }
    return lo;
}

template <typename T, int TAPS>
__global__ void __launch_bounds__(CI_THREADS) conv_attention_inputs_kernel(
    const T* proj, long long ld, const T* __restrict__ bias, const T* __restrict__ conv, int taps, const float* state,
    const T* __restrict__ q_norm_w, const T* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_sin, int rotary,
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* positions, const int* slot_map,
    const int* cu_seqlens, const int* seq_slots, const int* kv_lens, int B, int nq, int nkv, int D, int V, int Dp, int page_size,
    int write_kv, int head_norm) {
    extern __shared__ float y[];                       // [channels]
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int Cq = nq * D, Ck = write_kv ? nkv * D : 0, Cv = write_kv ? nkv * V : 0, C = Cq + Ck + Cv;
    const int p = __ldcg(positions + t);
    const int b = sequence_of(cu_seqlens, B, t);
    const int n_new = __ldcg(cu_seqlens + b + 1) - __ldcg(cu_seqlens + b);
    const int p0 = __ldcg(kv_lens + b) - n_new;        // position of the sequence's first token in this step
    const int slot = __ldcg(seq_slots + b);
    const float* hist = state + (size_t)slot * (taps > 1 ? taps - 1 : 0) * C;
    pdl_enter();
    // A channel's taps: all their loads (the rows they read, from the step's own projection or from the state, and their
    // weights) are issued before the first is used. With the number of taps known at compile time (TAPS >= 0) the loop
    // is unrolled and two channels are in flight per thread: a step of few tokens has nothing else to hide latency behind.
    float ssq = 0.f, ssk = 0.f;
    const int ntaps = TAPS >= 0 ? TAPS : taps;
    auto tap_input = [&](int c, int j, float bc) -> float {
        const int back = ntaps - 1 - j, pj = p - back;
        if (pj >= p0) return rnd<T>(to_f32(__ldcg(proj + (size_t)(t - back) * ld + c)) + bc);
        if (pj >= 0) return __ldcg(hist + (size_t)(ntaps - 1 - (p0 - pj)) * C + c);
        return 0.f;
    };
#pragma unroll 2
    for (int c = threadIdx.x; c < C; c += CI_THREADS) {
        const float bc = bias != nullptr ? to_f32(bias[c]) : 0.f;
        float acc;
        if (ntaps <= 0) {
            acc = rnd<T>(to_f32(__ldcg(proj + (size_t)t * ld + c)) + bc);
        } else if (TAPS > 0) {
            float u[TAPS > 0 ? TAPS : 1], w[TAPS > 0 ? TAPS : 1];
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                u[j] = tap_input(c, j, bc);
                w[j] = to_f32(conv[(size_t)c * TAPS + j]);
            }
            acc = 0.f;
#pragma unroll
            for (int j = 0; j < TAPS; ++j) acc = fmaf(w[j], u[j], acc);
            acc = rnd<T>(acc);
        } else {
            acc = 0.f;
            for (int j = 0; j < ntaps; ++j) acc = fmaf(to_f32(conv[(size_t)c * ntaps + j]), tap_input(c, j, bc), acc);
            acc = rnd<T>(acc);
        }
        y[c] = acc;
        if (c < Cq) ssq = fmaf(acc, acc, ssq);
        else if (c < Cq + Ck) ssk = fmaf(acc, acc, ssk);
    }
    if (head_norm) {
        // A warp per head: the order of a head's sum depends on the head's size alone.
        __syncthreads();
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int heads = nq + (write_kv ? nkv : 0);
        for (int hd = warp; hd < heads; hd += CI_THREADS / 32) {
            const T* w = hd < nq ? q_norm_w : k_norm_w;
            if (w == nullptr) continue;
            float* src = y + (size_t)hd * D;
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss = fmaf(src[d], src[d], ss);
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
            for (int d = lane; d < D; d += 32) src[d] = src[d] * inv * to_f32(w[d]);
        }
        q_norm_w = k_norm_w = nullptr;         // done; the whole-row norm below is skipped
    }
    float invq = 1.f, invk = 1.f;
    if (q_norm_w != nullptr) invq = 1.0f / sqrtf(block_sum(ssq, scratch) / (float)Cq + eps);
    if (k_norm_w != nullptr && write_kv) invk = 1.0f / sqrtf(block_sum(ssk, scratch) / (float)Ck + eps);
    __syncthreads();
    for (int c = threadIdx.x; c < Cq + Ck; c += CI_THREADS) {
        if (c < Cq) { if (q_norm_w != nullptr) y[c] = y[c] * invq * to_f32(q_norm_w[c]); }
        else if (k_norm_w != nullptr) y[c] = y[c] * invk * to_f32(k_norm_w[c - Cq]);
    }
    __syncthreads();
    const int half = rotary >> 1;
    const float* cs = cos_sin != nullptr ? cos_sin + (size_t)p * rotary : nullptr;       // [half][2] = (cos, sin)
    const int sm = write_kv ? __ldcg(slot_map + t) : 0;
    const int page = sm / page_size, off = sm - page * page_size;
    // Queries and keys: heads of Dp elements, the first D from y (rotated where the rotation reaches), zeros after.
    const int qk_heads = nq + (write_kv ? nkv : 0);
    for (int e = threadIdx.x; e < qk_heads * Dp; e += CI_THREADS) {
        const int head = e / Dp, d = e % Dp;
        float v = 0.f;
        if (d < D) {
            const float* src = y + (size_t)head * D;   // key heads follow the query heads in y
            v = src[d];
            if (cs != nullptr && d < rotary) {
                const int i = d < half ? d : d - half;
                const float other = d < half ? -src[d + half] : src[d - half];
                v = v * cs[2 * i] + other * cs[2 * i + 1];
            }
        }
        if (head < nq) q_out[((size_t)t * nq + head) * Dp + d] = from_f32<T>(v);
        else k_cache[(((size_t)page * nkv + head - nq) * page_size + off) * Dp + d] = from_f32<T>(v);
    }
    if (write_kv)
        for (int e = threadIdx.x; e < nkv * Dp; e += CI_THREADS) {
            const int head = e / Dp, d = e % Dp;
            v_cache[(((size_t)page * nkv + head) * page_size + off) * Dp + d] = from_f32<T>(d < V ? y[Cq + Ck + head * V + d] : 0.f);
        }
}

// proj [n, ld] of T: the step's projected rows, queries (nq * D) then, with write_kv, keys (nkv * D) and values (nkv * V);
// bias and conv [channels, taps] in the same channel order (null: none; taps 0: no convolution); state [slots, taps - 1, channels]
// float; cos_sin [positions, rotary / 2, 2] float (null: no rotation; pairs i, i + rotary / 2). head_norm: the norm weights are
// [D] and every head is normed by itself.
extern "C" int ti_conv_attention_inputs(const void* proj, long long ld, const void* bias, const void* conv, int taps, const float* state,
                                        const void* q_norm_w, const void* k_norm_w, float eps, const float* cos_sin, int rotary, void* q_out,
                                        void* k_cache, void* v_cache, const int* positions, const int* slot_map, const int* cu_seqlens,
                                        const int* seq_slots, const int* kv_lens, int n, int B, int nq, int nkv, int D, int V, int Dp,
                                        int page_size, int write_kv, int head_norm, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(taps >= 0 && taps <= CI_MAX_TAPS && (taps <= 1 || state != nullptr) && (taps == 0 || conv != nullptr), "conv_attention_inputs: %d taps", taps);
    TI_REQUIRE(D > 0 && V > 0 && Dp >= D && Dp >= V && nq > 0 && nkv > 0, "conv_attention_inputs: heads of %d / %d in rows of %d", D, V, Dp);
    TI_REQUIRE(cos_sin == nullptr || (rotary >= 2 && rotary % 2 == 0 && rotary <= D), "conv_attention_inputs: rotation over %d of %d", rotary, D);
    const int C = nq * D + (write_kv ? nkv * (D + V) : 0);
    const size_t smem = (size_t)C * sizeof(float);
    TI_REQUIRE(smem <= 160 * 1024, "conv_attention_inputs: %d channels", C);
#define CI_LAUNCH(TAPS)                                                                                                                       \
    do {                                                                                                                                      \
        if (smem > 48 * 1024) cudaFuncSetAttribute(conv_attention_inputs_kernel<T, TAPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        ti_launch(conv_attention_inputs_kernel<T, TAPS>, dim3(n), dim3(CI_THREADS), smem, stream, (const T*)proj, ld, (const T*)bias, (const T*)conv,  \
                  taps, state, (const T*)q_norm_w, (const T*)k_norm_w, eps, cos_sin, rotary, (T*)q_out, (T*)k_cache, (T*)v_cache, positions,       \
                  slot_map, cu_seqlens, seq_slots, kv_lens, B, nq, nkv, D, V, Dp, page_size, write_kv, head_norm);                               \
    } while (0)
    TI_DISPATCH_DTYPE(dtype, {
        switch (taps) {
            case 0: CI_LAUNCH(0); break;
            case 1: CI_LAUNCH(1); break;
            case 2: CI_LAUNCH(2); break;
            case 3: CI_LAUNCH(3); break;
            case 4: CI_LAUNCH(4); break;
            default: CI_LAUNCH(-1); break;
        }
    });
#undef CI_LAUNCH
    return ti_check_launch("conv_attention_inputs");
}

// After the step: the state of every sequence becomes the last taps - 1 rows u of the sequence (rows of this step where it
// brought enough, older ones moved up otherwise). A thread owns one channel of one sequence: it reads all it needs, then writes.
template <typename T>
__global__ void conv_state_update_kernel(float* state, const T* proj, long long ld, const T* __restrict__ bias, int taps, const int* cu_seqlens,
                                         const int* seq_slots, int C) {
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_enter();
    if (c >= C) return;
    const int t0 = __ldcg(cu_seqlens + b), n_new = __ldcg(cu_seqlens + b + 1) - t0;
    float* hist = state + (size_t)__ldcg(seq_slots + b) * (taps - 1) * C;
    const float bc = bias != nullptr ? to_f32(bias[c]) : 0.f;
    float keep[CI_MAX_TAPS];
#pragma unroll
    for (int i = 0; i < CI_MAX_TAPS - 1; ++i) {
        if (i >= taps - 1) break;
        const int r = n_new - (taps - 1) + i;          // row of this step, counted from the sequence's first new token
        keep[i] = r >= 0 ? rnd<T>(to_f32(__ldcg(proj + (size_t)(t0 + r) * ld + c)) + bc) : hist[(size_t)(taps - 1 + r) * C + c];
    }
#pragma unroll
    for (int i = 0; i < CI_MAX_TAPS - 1; ++i) {
        if (i >= taps - 1) break;
        hist[(size_t)i * C + c] = keep[i];
    }
}

extern "C" int ti_conv_state_update(float* state, const void* proj, long long ld, const void* bias, int taps, const int* cu_seqlens,
                                    const int* seq_slots, int B, int channels, int dtype, cudaStream_t stream) {
    if (B == 0 || taps <= 1) return 0;
    TI_REQUIRE(taps <= CI_MAX_TAPS && channels > 0 && B <= 65535, "conv_state_update: %d taps, %d channels, %d sequences", taps, channels, B);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(conv_state_update_kernel<T>, dim3((channels + 127) / 128, B), dim3(128), 0, stream, state, (const T*)proj, ld,
                                        (const T*)bias, taps, cu_seqlens, seq_slots, channels)));
    return ti_check_launch("conv_state_update");
}

// y [n, heads * V] = T(attn[n, heads, :V of Dp] * sigmoid(g [n, ldg])): the output gate, which also drops the rows' filling.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ y, const T* attn, const T* g, long long ldg, int heads, int V, int Dp, size_t count,
                                    int per_head) {
    pdl_enter();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / ((size_t)heads * V);
        const int c = (int)(i % ((size_t)heads * V)), head = c / V, d = c % V;
        float v = to_f32(__ldcg(attn + (t * heads + head) * Dp + d));
        if (g != nullptr) v = v / (1.0f + expf(-to_f32(__ldcg(g + t * ldg + (per_head ? head : c)))));
        y[i] = from_f32<T>(v);
    }
}

// The same with 16 bytes of outputs per thread.
template <typename T>
__global__ void sigmoid_gate_vec_kernel(T* __restrict__ y, const T* attn, const T* g, long long ldg, int heads, int V, int Dp, size_t vecs,
                                        int head_gate) {
    constexpr int N = Vec16<T>::N;
    const int per_head = V / N, per_row = heads * per_head;
    pdl_enter();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row;
        const int r = (int)(i % per_row), head = r / per_head, d = (r % per_head) * N;
        Vec16<T> a;
        a.load_cg(attn + (t * heads + head) * Dp + d);
        if (g != nullptr && head_gate) {         // one gate for the whole head: g [n, heads]
            const float s = 1.0f / (1.0f + expf(-to_f32(__ldcg(g + t * ldg + head))));
#pragma unroll
            for (int e = 0; e < N; ++e) a.v[e] *= s;
        } else if (g != nullptr) {
            Vec16<T> gate;
            gate.load_cg(g + t * ldg + head * V + d);
#pragma unroll
            for (int e = 0; e < N; ++e) a.v[e] = a.v[e] / (1.0f + expf(-gate.v[e]));
        }
        a.store(y + (t * heads + head) * V + d);
    }
}

// per_head: g is [n, heads] (rows ldg apart), one gate per head, instead of one per output element.
extern "C" int ti_sigmoid_gate(void* y, const void* attn, const void* g, long long ldg, int n, int heads, int V, int Dp, int per_head, int dtype,
                               cudaStream_t stream) {
    if (n == 0) return 0;
    TI_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        const bool vec = V % N == 0 && Dp % N == 0 && aligned16(y) && aligned16(attn) && (per_head || (ldg % N == 0 && aligned16(g)));
        const long long count = vec ? (long long)n * heads * (V / N) : (long long)n * heads * V;
        long long blocks = (count + 255) / 256;
        if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
        if (vec) ti_launch(sigmoid_gate_vec_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)y, (const T*)attn, (const T*)g, ldg, heads, V, Dp, (size_t)count, per_head);
        else ti_launch(sigmoid_gate_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)y, (const T*)attn, (const T*)g, ldg, heads, V, Dp, (size_t)count, per_head);
    });
    return ti_check_launch("sigmoid_gate");
}
