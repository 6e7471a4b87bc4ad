// Element-wise activations that are not a product's epilogue.
//
//   gelu                    y = T(gelu(x)), the exact form 0.5 x (1 + erf(x / sqrt 2)) or the tanh form
//                           0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))); the same kernel applies the squared rectifier
//                           max(x, 0)^2 (form 2) and tanh (form 3)
//   gated_token_embedding   g[t, j] = T(gelu_tanh(g[t, j]) * table[id[t], first + j]): a gate computed from the stream
//                           times the token's own vector, one slice of a table with a row per token id
//   gated_unit_limit        y[t, j] = T(a * sigmoid(slope * a) * (b + shift)), a = min(gu[t, j], limit),
//                           b = clamp(gu[t, ff + j], -limit, limit): a clamped gated unit from its fused gate|up product
#include "common.cuh"

#define ACT_GELU_ERF 0
#define ACT_GELU_TANH 1
#define ACT_RELU2 2
#define ACT_TANH 3

__device__ __forceinline__ float act_value(float z, int kind) {
    if (kind == ACT_RELU2) {
        const float r = fmaxf(z, 0.f);
        return r * r;
    }
    if (kind == ACT_TANH) return tanhf(z);
    return kind == ACT_GELU_TANH ? gelu_tanh_value(z) : gelu_erf_value(z);
}

template <typename T>
__global__ void gelu_kernel(T* out, const T* in, size_t count, int kind) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_enter();
    for (; i < count; i += stride) {
        const float z = to_f32(__ldcg(in + i));
        out[i] = from_f32<T>(act_value(z, kind));
    }
}

template <typename T>
__global__ void gelu_vec_kernel(T* out, const T* in, size_t vecs, int kind) {
    constexpr int N = Vec16<T>::N;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_enter();
    for (; i < vecs; i += stride) {
        Vec16<T> v;
        v.load_cg(in + i * N);
#pragma unroll
        for (int e = 0; e < N; ++e) v.v[e] = act_value(v.v[e], kind);
        v.store(out + i * N);
    }
}

extern "C" int ti_gelu(void* out, const void* in, long long count, int kind, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    TI_REQUIRE(kind >= ACT_GELU_ERF && kind <= ACT_TANH, "gelu: unknown form %d", kind);
    TI_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        const bool vec = count % N == 0 && aligned16(out) && aligned16(in);
        long long blocks = ((vec ? count / N : count) + 255) / 256;
        if (blocks > ti_sm_count() * 32) blocks = ti_sm_count() * 32;
        if (vec) ti_launch(gelu_vec_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)out, (const T*)in, (size_t)(count / N), kind);
        else ti_launch(gelu_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)out, (const T*)in, (size_t)count, kind);
    });
    return ti_check_launch("gelu");
}

template <typename T>
__global__ void gated_token_embedding_kernel(T* g, const T* __restrict__ table, const int* ids, int dim, int columns, int first,
                                             int vocab, size_t count) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_enter();
    for (; i < count; i += stride) {
        const int t = (int)(i / dim), j = (int)(i % dim);
        int id = __ldcg(ids + t);
        if (id < 0 || id >= vocab) id = 0;            // the embedding kernel has reported it
        const float e = to_f32(table[(size_t)id * columns + first + j]);
        g[i] = from_f32<T>(gelu_tanh_value(to_f32(__ldcg(g + i))) * e);
    }
}

extern "C" int ti_gated_token_embedding(void* g, const void* table, const int* ids, int n, int dim, int columns, int first, int vocab,
                                        int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(dim > 0 && first >= 0 && first + dim <= columns, "gated_token_embedding: columns [%d, %d) of %d", first, first + dim, columns);
    const long long count = (long long)n * dim;
    long long blocks = (count + 255) / 256;
    if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(gated_token_embedding_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)g, (const T*)table,
                                        ids, dim, columns, first, vocab, (size_t)count)));
    return ti_check_launch("gated_token_embedding");
}

// Rows in tiles that belong to units with limits of their own: `plan` [0] = tiles in use, [1 + t] = the unit of tile t
// (rows of tiles beyond those in use are left alone), `limits` [units]. Without a plan every row uses `limit`.
// A thread handles one 16-byte vector of outputs.
template <typename T>
__global__ void gated_unit_limit_kernel(T* __restrict__ y, const T* gu, int n, int ff, float limit, const int* plan, int tile,
                                        const float* __restrict__ limits, float slope, float shift) {
    constexpr int N = Vec16<T>::N;
    const int vecs = ff / N;
    pdl_enter();
    const int tiles = plan != nullptr ? __ldcg(plan) : 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n * vecs; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / vecs), j = (int)(i % vecs) * N;
        float lim = limit;
        if (plan != nullptr) {
            if (t / tile >= tiles) continue;
            lim = limits[__ldcg(plan + 1 + t / tile)];
        }
        Vec16<T> a, b;
        a.load_cg(gu + (size_t)t * 2 * ff + j);
        b.load_cg(gu + (size_t)t * 2 * ff + ff + j);
#pragma unroll
        for (int e = 0; e < N; ++e) {
            const float g = fminf(a.v[e], lim), u = fminf(fmaxf(b.v[e], -lim), lim);
            a.v[e] = g / (1.0f + __expf(-slope * g)) * (u + shift);
        }
        a.store(y + (size_t)t * ff + j);
    }
}

template <typename T>
__global__ void gated_unit_limit_scalar_kernel(T* __restrict__ y, const T* gu, int n, int ff, float limit, const int* plan, int tile,
                                               const float* __restrict__ limits, float slope, float shift) {
    pdl_enter();
    const int tiles = plan != nullptr ? __ldcg(plan) : 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n * ff; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / ff), j = (int)(i % ff);
        float lim = limit;
        if (plan != nullptr) {
            if (t / tile >= tiles) continue;
            lim = limits[__ldcg(plan + 1 + t / tile)];
        }
        const float g = fminf(to_f32(__ldcg(gu + (size_t)t * 2 * ff + j)), lim);
        const float u = fminf(fmaxf(to_f32(__ldcg(gu + (size_t)t * 2 * ff + ff + j)), -lim), lim);
        y[i] = from_f32<T>(g / (1.0f + expf(-slope * g)) * (u + shift));
    }
}

extern "C" int ti_gated_unit_limit(void* y, const void* gu, int n, int ff, float limit, const int* plan, int tile, const float* limits,
                                   float slope, float shift, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(ff > 0, "gated_unit_limit: size %d", ff);
    TI_REQUIRE(plan == nullptr || (tile > 0 && limits != nullptr), "gated_unit_limit: a plan needs its tile size and limits");
    TI_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        const bool vec = ff % N == 0 && aligned16(y) && aligned16(gu) && sizeof(T) == 2;      // the 32-bit path keeps expf
        const long long count = vec ? (long long)n * (ff / N) : (long long)n * ff;
        long long blocks = (count + 255) / 256;
        if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
        if (vec) ti_launch(gated_unit_limit_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)y, (const T*)gu, n, ff, limit, plan, tile, limits, slope, shift);
        else ti_launch(gated_unit_limit_scalar_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)y, (const T*)gu, n, ff, limit, plan, tile, limits, slope, shift);
    });
    return ti_check_launch("gated_unit_limit");
}

// A gated unit's inner activation without a clamp: y[t, j] = act(gu[t, j]) * gu[t, ff + j], act = SiLU (kind 0) or the tanh
// form of GELU (kind 1); gate rows first, then up rows. 32-bit arithmetic, one rounding.
template <typename T>
__global__ void gated_act_kernel(T* __restrict__ y, const T* gu, int ff, int kind, size_t count) {
    pdl_enter();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / ff;
        const int j = (int)(i % ff);
        const float g = to_f32(__ldcg(gu + t * 2 * ff + j)), u = to_f32(__ldcg(gu + t * 2 * ff + ff + j));
        const float a = kind == 1 ? gelu_tanh_value(g) : g / (1.0f + expf(-g));
        y[i] = from_f32<T>(a * u);
    }
}

// The same with 16 bytes of outputs per thread.
template <typename T>
__global__ void gated_act_vec_kernel(T* __restrict__ y, const T* gu, int ff, int kind, size_t vecs) {
    constexpr int N = Vec16<T>::N;
    const int per_row = ff / N;
    pdl_enter();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row;
        const int j = (int)(i % per_row) * N;
        Vec16<T> g, u;
        g.load_cg(gu + t * 2 * ff + j);
        u.load_cg(gu + t * 2 * ff + ff + j);
#pragma unroll
        for (int e = 0; e < N; ++e) g.v[e] = (kind == 1 ? gelu_tanh_value(g.v[e]) : g.v[e] / (1.0f + expf(-g.v[e]))) * u.v[e];
        g.store(y + t * ff + j);
    }
}

extern "C" int ti_gated_act(void* y, const void* gu, int n, int ff, int kind, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(ff > 0 && (kind == 0 || kind == 1), "gated_act: size %d, kind %d", ff, kind);
    TI_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        const bool vec = ff % N == 0 && aligned16(y) && aligned16(gu);
        const long long count = vec ? (long long)n * (ff / N) : (long long)n * ff;
        long long blocks = (count + 255) / 256;
        if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
        if (vec) ti_launch(gated_act_vec_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)y, (const T*)gu, ff, kind, (size_t)count);
        else ti_launch(gated_act_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)y, (const T*)gu, ff, kind, (size_t)count);
    });
    return ti_check_launch("gated_act");
}
