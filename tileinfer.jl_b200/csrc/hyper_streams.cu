// Several copies of the residual stream (hyper-connections), kept in 32-bit: x [n][S][size].
//
// A sublayer reads u = sum_s a[s] x_s through a layer norm (weight, optional bias); its output y [n][size] is written back to all
// copies at once from the old ones:  x_t <- sum_s M[s][t] x_s + m * c[t] * y  (M indexed [from][to]). The kernel that writes a
// sublayer's output back also makes the next reader's input: u' = sum_t a'[t] x_t of the new copies, normed and rounded once.
// With S = 1, M = [[1]], a = c = [1] this is the plain residual sum x += m y followed by the next norm, so one kernel serves
// both arrangements. One block per token; everything is 32-bit arithmetic until the one rounding of the reader's input.
#include "common.cuh"

#define HS_MAX_STREAMS 8

static int hs_threads(int size) { return size >= 4096 ? 512 : size >= 1024 ? 256 : 128; }

// x [n][S][size] <- x0 [n][size] in every copy.
__global__ void streams_begin_kernel(float* __restrict__ x, const float* x0, int S, int size, size_t count) {
    pdl_enter();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / size;
        const int c = (int)(i % size);
        const float v = __ldcg(x0 + i);
        for (int s = 0; s < S; ++s) x[(t * S + s) * size + c] = v;
    }
}

extern "C" int ti_streams_begin(float* x, const float* x0, int n, int S, int size, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(S >= 1 && S <= HS_MAX_STREAMS && size > 0, "streams_begin: %d copies of rows of %d", S, size);
    const size_t count = (size_t)n * size;
    long long blocks = (count + 255) / 256;
    if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
    ti_launch(streams_begin_kernel, dim3((int)blocks), dim3(256), 0, stream, x, x0, S, size, count);
    return ti_check_launch("streams_begin");
}

struct StreamTables {
    float mix[HS_MAX_STREAMS * HS_MAX_STREAMS];   // [from][to]
    float out[HS_MAX_STREAMS];                     // m * c[t]
    float in_next[HS_MAX_STREAMS];                 // a'[t]
};

// The layer norm of `row_u` [size] (shared memory; a thread reads back the elements it wrote) into dst.
template <typename T>
__device__ __forceinline__ void norm_row(T* __restrict__ dst, const float* row_u, float sum, const T* __restrict__ w, const T* __restrict__ b,
                                         float eps, int centred, int size, float* scratch) {
    float mean = 0.f;
    if (centred) mean = block_sum(sum, scratch) / (float)size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float d = row_u[i] - mean;
        ss = fmaf(d, d, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float v = (row_u[i] - mean) * inv * to_f32(w[i]);
        if (b != nullptr) v += to_f32(b[i]);
        dst[i] = from_f32<T>(v);
    }
}

// h = norm(sum_s a[s] x_s): the first reader's input (nothing to write back yet).
template <typename T>
__global__ void streams_read_norm_kernel(T* __restrict__ h, const float* x, const float* __restrict__ a, int S, const T* __restrict__ w,
                                         const T* __restrict__ b, float eps, int centred, int size) {
    extern __shared__ float row_u[];
    __shared__ float scratch[33];
    const float* rows = x + (size_t)blockIdx.x * S * size;
    pdl_enter();
    float sum = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float u = 0.f;
        for (int s = 0; s < S; ++s) u = fmaf(a[s], __ldcg(rows + (size_t)s * size + i), u);
        row_u[i] = u;
        sum += u;
    }
    norm_row<T>(h + (size_t)blockIdx.x * size, row_u, sum, w, b, eps, centred, size, scratch);
}

// Write a sublayer's output back and make the next reader's input. The output is `delta` [n][size] of T, or the sum of
// `n_partials` 32-bit arrays [n][size] `partial_stride` apart (a product cut over k, or one unrounded 32-bit result).
template <typename T>
__global__ void streams_update_kernel(float* x, const T* delta, const float* partials, int n_partials, size_t partial_stride, StreamTables tab,
                                      int S, T* __restrict__ h, const T* __restrict__ w, const T* __restrict__ b, float eps, int centred, int size) {
    extern __shared__ float row_u[];
    __shared__ float scratch[33];
    float* rows = x + (size_t)blockIdx.x * S * size;
    pdl_enter();
    float sum = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float y;
        if (partials != nullptr) {
            const float* p = partials + (size_t)blockIdx.x * size + i;
            y = __ldcg(p);
            for (int s = 1; s < n_partials; ++s) y += __ldcg(p + (size_t)s * partial_stride);
        } else {
            y = to_f32(__ldcg(delta + (size_t)blockIdx.x * size + i));
        }
        float old[HS_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HS_MAX_STREAMS; ++s) old[s] = s < S ? __ldcg(rows + (size_t)s * size + i) : 0.f;
        float u = 0.f;
#pragma unroll
        for (int t = 0; t < HS_MAX_STREAMS; ++t) {
            if (t >= S) break;
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < HS_MAX_STREAMS; ++s)
                if (s < S) v = fmaf(tab.mix[s * HS_MAX_STREAMS + t], old[s], v);
            v = fmaf(tab.out[t], y, v);
            rows[(size_t)t * size + i] = v;
            u = fmaf(tab.in_next[t], v, u);
        }
        row_u[i] = u;
        sum += u;
    }
    if (h == nullptr) return;
    norm_row<T>(h + (size_t)blockIdx.x * size, row_u, sum, w, b, eps, centred, size, scratch);
}

extern "C" int ti_streams_read_norm(void* h, const float* x, const float* a, int S, const void* w, const void* b, float eps, int centred, int n,
                                    int size, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(S >= 1 && S <= HS_MAX_STREAMS && size > 0, "streams_read_norm: %d copies of rows of %d", S, size);
    const size_t smem = (size_t)size * sizeof(float);
    TI_REQUIRE(smem <= 160 * 1024, "streams_read_norm: rows of %d", size);
    TI_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_read_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ti_launch(streams_read_norm_kernel<T>, dim3(n), dim3(hs_threads(size)), smem, stream, (T*)h, x, a, S, (const T*)w, (const T*)b, eps, centred, size);
    });
    return ti_check_launch("streams_read_norm");
}

// mix [S][S] (from, to), out [S] (already times the multiplier), in_next [S]: host arrays, passed by value.
extern "C" int ti_streams_update(float* x, const void* delta, const float* partials, int n_partials, long long partial_stride, const float* mix,
                                 const float* out, const float* in_next, int S, void* h, const void* w, const void* b, float eps, int centred,
                                 int n, int size, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(S >= 1 && S <= HS_MAX_STREAMS && size > 0, "streams_update: %d copies of rows of %d", S, size);
    TI_REQUIRE((delta != nullptr) != (partials != nullptr && n_partials > 0), "streams_update: rows or partial sums, one of them");
    StreamTables tab = {};
    for (int s = 0; s < S; ++s) {
        for (int t = 0; t < S; ++t) tab.mix[s * HS_MAX_STREAMS + t] = mix[s * S + t];
        tab.out[s] = out[s];
        tab.in_next[s] = in_next != nullptr ? in_next[s] : 0.f;
    }
    const size_t smem = (size_t)size * sizeof(float);
    TI_REQUIRE(smem <= 160 * 1024, "streams_update: rows of %d", size);
    TI_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_update_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ti_launch(streams_update_kernel<T>, dim3(n), dim3(hs_threads(size)), smem, stream, x, (const T*)delta, partials, n_partials,
                  (size_t)partial_stride, tab, S, (T*)h, (const T*)w, (const T*)b, eps, centred, size);
    });
    return ti_check_launch("streams_update");
}
