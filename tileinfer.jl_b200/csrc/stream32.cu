// A residual stream kept in 32-bit, whatever the element type T of the activations and weights is.
//
//   embed_positions32   x = E[id] + P[position]                                  (both tables in T, the sum in 32-bit)
//   embed_bigram32      x = E[id] * scale + G[(previous id * a + id * b) mod buckets]   (the row `buckets` for a sequence's first token)
//   cast_rows           h = T(x)                                                    (h's rows may be longer than x's)
//   norm32              y = T(x / rms(x) * g(w)),  x in 32-bit or in T
//   branch_norm_add32   x += mult * d / rms(d) * g(w);  then  h = T(x)  or  h = T(x / rms(x) * g_out(w_out))
//   sum_add_norm32      x += d1 + d2;  then  h = T(x / rms(x) * g_out(w_out))       (two sublayers that read the same input)
//
// rms(v) = sqrt(mean(v^2) + eps); g(w) = w, or 1 + w where the checkpoint keeps the gain minus one ("offset"). A norm's flags
// word carries that choice in bit 0 and, in bit 1, "centred": the row's mean is taken off first and rms is then the root of the
// mean squared deviation (a layer norm with a weight and no bias). branch_norm_add32 may add a bias vector to d first. Everything
// between the loads and the one rounding on store is 32-bit. d is a sublayer's output: [n, size] in T, or the
// 32-bit partial sums [s, n, size] of a product that was cut over k (added in split order, not rounded).
// One block per row; the order of a row's sums depends on the row's size alone.
#include "common.cuh"

template <typename T>
__global__ void embed_positions32_kernel(float* __restrict__ x, const T* __restrict__ table, const T* __restrict__ pos_table,
                                         const int* ids, const int* positions, int hidden, int vocab, int max_positions,
                                         int* __restrict__ status) {
    const int t = blockIdx.x;
    pdl_enter();
    int id = __ldcg(ids + t), p = __ldcg(positions + t);
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(status, 1 + t);
        id = 0;
    }
    if (p < 0 || p >= max_positions) {
        if (threadIdx.x == 0) atomicExch(status, 1 + t);
        p = 0;
    }
    const T* e = table + (size_t)id * hidden;
    const T* q = pos_table + (size_t)p * hidden;
    float* dst = x + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = pos_table != nullptr ? to_f32(e[i]) + to_f32(q[i]) : to_f32(e[i]);
}

extern "C" int ti_embed_positions32(float* x, const void* table, const void* pos_table, const int* ids, const int* positions,
                                    int n_tokens, int hidden, int vocab, int max_positions, int dtype, int* status,
                                    cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    if (pos_table == nullptr) max_positions = 1 << 30;          // no position table: the token's row alone
    TI_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0 && max_positions > 0, "embed_positions32: bad sizes n=%d hidden=%d vocab=%d positions=%d",
               n_tokens, hidden, vocab, max_positions);
    const int threads = hidden >= 1024 ? 256 : 128;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(embed_positions32_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, x, (const T*)table,
                                        (const T*)pos_table, ids, positions, hidden, vocab, max_positions, status)));
    return ti_check_launch("embed_positions32");
}

// A token embedding times a constant plus a row of a second table chosen by a hash of the token and the token before it in
// its sequence. The token before comes from the step itself, or, where the step begins in the middle of a sequence, from `last`
// [slots]: the last token that earlier steps ran, which last_token_update writes after this kernel (a launch of its own,
// since these blocks read what it overwrites). A sequence's first token takes the table's extra row `buckets`. pair == null: no
// second table.
template <typename T>
__global__ void embed_bigram32_kernel(float* __restrict__ x, const T* __restrict__ table, const T* __restrict__ pair, const int* ids,
                                      const int* positions, const int* tok_slot, const int* last, int hidden, int vocab, float scale,
                                      long long buckets, long long mul_prev, long long mul_cur, int* __restrict__ status) {
    const int t = blockIdx.x;
    pdl_enter();
    int id = __ldcg(ids + t);
    const int p = __ldcg(positions + t);
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(status, 1 + t);
        id = 0;
    }
    const T* g = nullptr;
    if (pair != nullptr) {
        long long row = buckets;
        if (p > 0) {
            const int slot = __ldcg(tok_slot + t);
            int prev;
            if (t > 0 && __ldcg(tok_slot + t - 1) == slot && __ldcg(positions + t - 1) == p - 1) prev = __ldcg(ids + t - 1);
            else prev = __ldcg(last + slot);
            if (prev < 0 || prev >= vocab) prev = 0;
            row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
            if (row < 0) row += buckets;
        }
        g = pair + (size_t)row * hidden;
    }
    const T* e = table + (size_t)id * hidden;
    float* dst = x + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_f32(e[i]) * scale;
        dst[i] = g != nullptr ? v + to_f32(g[i]) : v;
    }
}

extern "C" int ti_embed_bigram32(float* x, const void* table, const void* pair, const int* ids, const int* positions, const int* tok_slot,
                                 const int* last, int n_tokens, int hidden, int vocab, float scale, long long buckets, long long mul_prev,
                                 long long mul_cur, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    TI_REQUIRE(hidden > 0 && vocab > 0 && (pair == nullptr || (buckets > 0 && last != nullptr)), "embed_bigram32: hidden %d vocab %d buckets %lld",
               hidden, vocab, buckets);
    const int threads = hidden >= 1024 ? 256 : 128;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(embed_bigram32_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, x, (const T*)table, (const T*)pair, ids,
                                        positions, tok_slot, last, hidden, vocab, scale, buckets, mul_prev, mul_cur, status)));
    return ti_check_launch("embed_bigram32");
}

__global__ void last_token_update_kernel(int* last, const int* ids, const int* cu_seqlens, const int* seq_slots, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_enter();
    if (b < B) last[__ldcg(seq_slots + b)] = __ldcg(ids + __ldcg(cu_seqlens + b + 1) - 1);
}

extern "C" int ti_last_token_update(int* last, const int* ids, const int* cu_seqlens, const int* seq_slots, int B, cudaStream_t stream) {
    if (B == 0) return 0;
    ti_launch(last_token_update_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, last, ids, cu_seqlens, seq_slots, B);
    return ti_check_launch("last_token_update");
}

// h [n, ldh] (the first `size` elements of every row) = T(x [n, size]).
template <typename T>
__global__ void cast_rows_ld_kernel(T* __restrict__ h, long long ldh, const float* x, int size, size_t count) {
    pdl_enter();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / size;
        h[t * ldh + (i - t * size)] = from_f32<T>(__ldcg(x + i));
    }
}

extern "C" int ti_cast_rows_ld(void* h, long long ldh, const float* x, int n, int size, int dtype, cudaStream_t stream) {
    const long long count = (long long)n * size;
    if (count == 0) return 0;
    TI_REQUIRE(ldh >= size, "cast_rows_ld: rows of %d in a buffer with rows of %lld", size, ldh);
    long long blocks = (count + 255) / 256;
    if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(cast_rows_ld_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)h, ldh, x, size, (size_t)count)));
    return ti_check_launch("cast_rows_ld");
}

template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ h, const float* x, size_t count) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_enter();
    for (; i < count; i += stride) h[i] = from_f32<T>(__ldcg(x + i));
}

extern "C" int ti_cast_rows(void* h, const float* x, long long count, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    long long blocks = (count + 255) / 256;
    if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(cast_rows_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)h, x, (size_t)count)));
    return ti_check_launch("cast_rows");
}

// Threads of the row kernels: a function of the row's size alone.
static int row_threads(int size) { return size >= 4096 ? 512 : size >= 1024 ? 256 : 128; }

template <typename T, typename X>
__global__ void norm32_kernel(T* __restrict__ y, const X* x, const T* __restrict__ w, int size, float eps, int offset) {
    __shared__ float scratch[33];
    const X* row = x + (size_t)blockIdx.x * size;
    T* dst = y + (size_t)blockIdx.x * size;
    float ss = 0.f, mean = 0.f;
    pdl_enter();
    if (offset & 2) {
        float s = 0.f;
        for (int i = threadIdx.x; i < size; i += blockDim.x) s += to_f32(__ldcg(row + i));
        mean = block_sum(s, scratch) / (float)size;
    }
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = to_f32(__ldcg(row + i)) - mean;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float g = (offset & 1) ? 1.0f + to_f32(w[i]) : to_f32(w[i]);
        dst[i] = from_f32<T>((to_f32(__ldcg(row + i)) - mean) * inv * g);
    }
}

extern "C" int ti_norm32(void* y, const void* x, int x_is_f32, const void* w, int n_rows, int size, float eps, int offset,
                         int dtype, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(size > 0, "norm32: size %d", size);
    const int threads = row_threads(size);
    TI_DISPATCH_DTYPE(dtype, {
        if (x_is_f32) ti_launch(norm32_kernel<T, float>, dim3(n_rows), dim3(threads), 0, stream, (T*)y, (const float*)x, (const T*)w, size, eps, offset);
        else ti_launch(norm32_kernel<T, T>, dim3(n_rows), dim3(threads), 0, stream, (T*)y, (const T*)x, (const T*)w, size, eps, offset);
    });
    return ti_check_launch("norm32");
}

// `gather` [n, per_row]: the branch's row is the sum, in that order and in 32-bit, of the rows gather[row][0 .. per_row) of
// `delta` (the outputs of the units a token went through), instead of row `row` of `delta`.
template <typename T>
__global__ void branch_norm_add32_kernel(float* x, const T* delta, const float* partials, int n_partials, size_t partial_stride,
                                         const int* gather, int per_row, const T* __restrict__ dbias, const T* __restrict__ w, int offset, float eps,
                                         float mult, T* __restrict__ h, const T* __restrict__ w_out, int offset_out, float eps_out, int size) {
    extern __shared__ float row_d[];           // [size]: the branch's row, then the stream's new row
    __shared__ float scratch[33];
    float* row = x + (size_t)blockIdx.x * size;
    float ss = 0.f, sum = 0.f;
    pdl_enter();
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float d;
        if (partials != nullptr) {
            const float* p = partials + (size_t)blockIdx.x * size + i;
            d = __ldcg(p);
            for (int s = 1; s < n_partials; ++s) d += __ldcg(p + (size_t)s * partial_stride);
        } else if (gather != nullptr) {
            d = 0.f;
            for (int j = 0; j < per_row; ++j)
                d += to_f32(__ldcg(delta + (size_t)__ldcg(gather + (size_t)blockIdx.x * per_row + j) * size + i));
        } else {
            d = to_f32(__ldcg(delta + (size_t)blockIdx.x * size + i));
        }
        if (dbias != nullptr) d += to_f32(dbias[i]);
        row_d[i] = d;
        ss = fmaf(d, d, ss);
        sum += d;
    }
    float mean = 0.f;
    if (offset & 2) {                          // centred: the squared deviations need the mean first (a thread reads back its own elements)
        mean = block_sum(sum, scratch) / (float)size;
        ss = 0.f;
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            const float d = row_d[i] - mean;
            ss = fmaf(d, d, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    float ss2 = 0.f, sum2 = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float g = (offset & 1) ? 1.0f + to_f32(w[i]) : to_f32(w[i]);
        const float v = __ldcg(row + i) + mult * ((row_d[i] - mean) * inv * g);
        row[i] = v;
        row_d[i] = v;                         // the same thread reads it back below
        ss2 = fmaf(v, v, ss2);
        sum2 += v;
    }
    if (h == nullptr) return;
    T* dst = h + (size_t)blockIdx.x * size;
    if (w_out == nullptr) {
        for (int i = threadIdx.x; i < size; i += blockDim.x) dst[i] = from_f32<T>(row_d[i]);
        return;
    }
    float mean2 = 0.f;
    if (offset_out & 2) {
        mean2 = block_sum(sum2, scratch) / (float)size;
        ss2 = 0.f;
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            const float d = row_d[i] - mean2;
            ss2 = fmaf(d, d, ss2);
        }
    }
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)size + eps_out);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float g = (offset_out & 1) ? 1.0f + to_f32(w_out[i]) : to_f32(w_out[i]);
        dst[i] = from_f32<T>((row_d[i] - mean2) * inv2 * g);
    }
}

// The same for bfloat16 rows with four elements per thread and step: 16-byte accesses of the 32-bit stream, 8-byte
// accesses of the bfloat16 rows. The order of a row's sums still depends on the row's size alone.
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
    const uint2 t = __ldcg(reinterpret_cast<const uint2*>(p));
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void load4w(const bf16* __restrict__ p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&a), *reinterpret_cast<const unsigned*>(&b));
}

__global__ void branch_norm_add32_vec_kernel(float* x, const bf16* delta, const float* partials, int n_partials, size_t partial_stride,
                                             const int* gather, int per_row, const bf16* __restrict__ dbias, const bf16* __restrict__ w, int offset,
                                             float eps, float mult, bf16* __restrict__ h, const bf16* __restrict__ w_out, int offset_out, float eps_out,
                                             int size) {
    extern __shared__ float row_d[];
    __shared__ float scratch[33];
    float* row = x + (size_t)blockIdx.x * size;
    float ss = 0.f, sum = 0.f;
    pdl_enter();
    for (int i = threadIdx.x * 4; i < size; i += blockDim.x * 4) {
        float d[4];
        if (partials != nullptr) {
            const float* p = partials + (size_t)blockIdx.x * size + i;
            float4 t = __ldcg(reinterpret_cast<const float4*>(p));
            d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
            for (int s = 1; s < n_partials; ++s) {
                t = __ldcg(reinterpret_cast<const float4*>(p + (size_t)s * partial_stride));
                d[0] += t.x; d[1] += t.y; d[2] += t.z; d[3] += t.w;
            }
        } else if (gather != nullptr) {
            d[0] = d[1] = d[2] = d[3] = 0.f;
            for (int j = 0; j < per_row; ++j) {
                float v[4];
                load4(delta + (size_t)__ldcg(gather + (size_t)blockIdx.x * per_row + j) * size + i, v);
                d[0] += v[0]; d[1] += v[1]; d[2] += v[2]; d[3] += v[3];
            }
        } else {
            load4(delta + (size_t)blockIdx.x * size + i, d);
        }
        if (dbias != nullptr) {
            float b[4];
            load4w(dbias + i, b);
#pragma unroll
            for (int e = 0; e < 4; ++e) d[e] += b[e];
        }
        *reinterpret_cast<float4*>(row_d + i) = make_float4(d[0], d[1], d[2], d[3]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            ss = fmaf(d[e], d[e], ss);
            sum += d[e];
        }
    }
    float mean = 0.f;
    if (offset & 2) {
        mean = block_sum(sum, scratch) / (float)size;
        ss = 0.f;
        for (int i = threadIdx.x * 4; i < size; i += blockDim.x * 4) {
            const float4 t = *reinterpret_cast<const float4*>(row_d + i);
            const float d[4] = {t.x - mean, t.y - mean, t.z - mean, t.w - mean};
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(d[e], d[e], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    float ss2 = 0.f, sum2 = 0.f;
    for (int i = threadIdx.x * 4; i < size; i += blockDim.x * 4) {
        float g[4];
        load4w(w + i, g);
        const float4 xv = __ldcg(reinterpret_cast<const float4*>(row + i));
        const float4 dv = *reinterpret_cast<const float4*>(row_d + i);
        const float xs[4] = {xv.x, xv.y, xv.z, xv.w}, ds[4] = {dv.x, dv.y, dv.z, dv.w};
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            v[e] = xs[e] + mult * ((ds[e] - mean) * inv * ((offset & 1) ? 1.0f + g[e] : g[e]));
            ss2 = fmaf(v[e], v[e], ss2);
            sum2 += v[e];
        }
        *reinterpret_cast<float4*>(row + i) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(row_d + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
    if (h == nullptr) return;
    bf16* dst = h + (size_t)blockIdx.x * size;
    float inv2 = 1.0f, mean2 = 0.f;
    if (w_out != nullptr) {
        if (offset_out & 2) {
            mean2 = block_sum(sum2, scratch) / (float)size;
            ss2 = 0.f;
            for (int i = threadIdx.x * 4; i < size; i += blockDim.x * 4) {
                const float4 t = *reinterpret_cast<const float4*>(row_d + i);
                const float d[4] = {t.x - mean2, t.y - mean2, t.z - mean2, t.w - mean2};
#pragma unroll
                for (int e = 0; e < 4; ++e) ss2 = fmaf(d[e], d[e], ss2);
            }
        }
        ss2 = block_sum(ss2, scratch);
        inv2 = 1.0f / sqrtf(ss2 / (float)size + eps_out);
    }
    for (int i = threadIdx.x * 4; i < size; i += blockDim.x * 4) {
        const float4 t = *reinterpret_cast<const float4*>(row_d + i);
        float v[4] = {t.x, t.y, t.z, t.w};
        if (w_out != nullptr) {
            float g[4];
            load4w(w_out + i, g);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = (v[e] - mean2) * inv2 * ((offset_out & 1) ? 1.0f + g[e] : g[e]);
        }
        store4(dst + i, v);
    }
}

extern "C" int ti_branch_norm_add32(float* x, const void* delta, const float* partials, int n_partials, long long partial_stride,
                                    const int* gather, int per_row, const void* dbias, const void* w, int offset, float eps, float mult, void* h,
                                    const void* w_out, int offset_out, float eps_out, int n_rows, int size, int dtype, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(size > 0 && size <= 50000, "branch_norm_add32: size %d", size);
    TI_REQUIRE((delta != nullptr) != (partials != nullptr), "branch_norm_add32: give delta or partials, not both");
    TI_REQUIRE(partials == nullptr || n_partials >= 1, "branch_norm_add32: n_partials %d", n_partials);
    TI_REQUIRE(gather == nullptr || (delta != nullptr && per_row >= 1), "branch_norm_add32: gathered rows need delta and a count");
    const int threads = row_threads(size);
    const size_t smem = (size_t)size * sizeof(float);
    TI_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) {
            static bool raised = false;       // per element type (this block is instantiated once for each)
            if (!raised) {
                cudaFuncSetAttribute(branch_norm_add32_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
                raised = true;
            }
        }
        const bool vec = sizeof(T) == 2 && size % 4 == 0 && smem <= 48 * 1024 && aligned16(x) && (partials == nullptr || (aligned16(partials) && partial_stride % 4 == 0)) &&
                         (((uintptr_t)delta | (uintptr_t)dbias | (uintptr_t)w | (uintptr_t)h | (uintptr_t)w_out) & 7) == 0;
        if (vec) {
            const int vt = size >= 2048 ? 256 : 128;
            ti_launch(branch_norm_add32_vec_kernel, dim3(n_rows), dim3(vt), smem, stream, x, (const bf16*)delta, partials, n_partials,
                      (size_t)partial_stride, gather, per_row, (const bf16*)dbias, (const bf16*)w, offset, eps, mult, (bf16*)h, (const bf16*)w_out,
                      offset_out, eps_out, size);
        } else
        ti_launch(branch_norm_add32_kernel<T>, dim3(n_rows), dim3(threads), smem, stream, x, (const T*)delta, partials, n_partials,
                  (size_t)partial_stride, gather, per_row, (const T*)dbias, (const T*)w, offset, eps, mult, (T*)h, (const T*)w_out, offset_out, eps_out,
                  size);
    });
    return ti_check_launch("branch_norm_add32");
}

// Two sublayers read the same normed input and both are added: x += d1 + d2 (d2 may be absent), the sum in 32-bit, then the
// next reader's input h = T(x / rms(x) * g(w_out)). d1, d2: rows [n, size] of T, or 32-bit partial sums [s, n, size].
template <typename T>
__device__ __forceinline__ float branch_value(const T* d, const float* partials, int n_partials, size_t stride, size_t at) {
    if (partials != nullptr) {
        float v = __ldcg(partials + at);
        for (int s = 1; s < n_partials; ++s) v += __ldcg(partials + (size_t)s * stride + at);
        return v;
    }
    return d != nullptr ? to_f32(__ldcg(d + at)) : 0.f;
}

template <typename T>
__global__ void sum_add_norm32_kernel(float* x, const T* d1, const float* p1, int n1, size_t s1, const T* d2, const float* p2, int n2, size_t s2,
                                      T* __restrict__ h, const T* __restrict__ w_out, int offset_out, float eps_out, int size) {
    extern __shared__ float row_d[];
    __shared__ float scratch[33];
    float* row = x + (size_t)blockIdx.x * size;
    float ss = 0.f;
    pdl_enter();
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const size_t at = (size_t)blockIdx.x * size + i;
        const float v = __ldcg(row + i) + (branch_value(d1, p1, n1, s1, at) + branch_value(d2, p2, n2, s2, at));
        row[i] = v;
        row_d[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (h == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps_out);
    T* dst = h + (size_t)blockIdx.x * size;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float g = offset_out ? 1.0f + to_f32(w_out[i]) : to_f32(w_out[i]);
        dst[i] = from_f32<T>(row_d[i] * inv * g);
    }
}

// The same for bfloat16 rows with four elements per thread and step (16-byte accesses of the stream and of partial sums, 8-byte
// accesses of the rows); the sums in the same order.
__device__ __forceinline__ void branch_value4(const bf16* d, const float* partials, int n_partials, size_t stride, size_t at, float (&v)[4]) {
    if (partials != nullptr) {
        float4 t = __ldcg(reinterpret_cast<const float4*>(partials + at));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        for (int s = 1; s < n_partials; ++s) {
            t = __ldcg(reinterpret_cast<const float4*>(partials + (size_t)s * stride + at));
            v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
        }
    } else if (d != nullptr) {
        load4(d + at, v);
    } else {
        v[0] = v[1] = v[2] = v[3] = 0.f;
    }
}

__global__ void sum_add_norm32_vec_kernel(float* x, const bf16* d1, const float* p1, int n1, size_t s1, const bf16* d2, const float* p2, int n2,
                                          size_t s2, bf16* __restrict__ h, const bf16* __restrict__ w_out, int offset_out, float eps_out, int size) {
    extern __shared__ float row_d[];
    __shared__ float scratch[33];
    float* row = x + (size_t)blockIdx.x * size;
    float ss = 0.f;
    pdl_enter();
    for (int i = threadIdx.x * 4; i < size; i += blockDim.x * 4) {
        const size_t at = (size_t)blockIdx.x * size + i;
        float a[4], b[4];
        branch_value4(d1, p1, n1, s1, at, a);
        branch_value4(d2, p2, n2, s2, at, b);
        const float4 xv = __ldcg(reinterpret_cast<const float4*>(row + i));
        const float v[4] = {xv.x + (a[0] + b[0]), xv.y + (a[1] + b[1]), xv.z + (a[2] + b[2]), xv.w + (a[3] + b[3])};
        *reinterpret_cast<float4*>(row + i) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(row_d + i) = make_float4(v[0], v[1], v[2], v[3]);
#pragma unroll
        for (int e = 0; e < 4; ++e) ss = fmaf(v[e], v[e], ss);
    }
    if (h == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps_out);
    bf16* dst = h + (size_t)blockIdx.x * size;
    for (int i = threadIdx.x * 4; i < size; i += blockDim.x * 4) {
        const float4 t = *reinterpret_cast<const float4*>(row_d + i);
        float g[4], v[4] = {t.x, t.y, t.z, t.w};
        load4w(w_out + i, g);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = v[e] * inv * (offset_out ? 1.0f + g[e] : g[e]);
        store4(dst + i, v);
    }
}

extern "C" int ti_sum_add_norm32(float* x, const void* d1, const float* p1, int n1, long long s1, const void* d2, const float* p2, int n2, long long s2,
                                 void* h, const void* w_out, int offset_out, float eps_out, int n_rows, int size, int dtype, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(size > 0 && size <= 50000, "sum_add_norm32: size %d", size);
    TI_REQUIRE((d1 != nullptr) != (p1 != nullptr) && !(d2 != nullptr && p2 != nullptr), "sum_add_norm32: every branch is rows or partial sums");
    TI_REQUIRE(h == nullptr || w_out != nullptr, "sum_add_norm32: the next input needs its norm's weight");
    const size_t smem = (size_t)size * sizeof(float);
    TI_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(sum_add_norm32_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        const bool vec = sizeof(T) == 2 && size % 4 == 0 && smem <= 48 * 1024 && aligned16(x) && (p1 == nullptr || (aligned16(p1) && s1 % 4 == 0)) &&
                         (p2 == nullptr || (aligned16(p2) && s2 % 4 == 0)) &&
                         (((uintptr_t)d1 | (uintptr_t)d2 | (uintptr_t)h | (uintptr_t)w_out) & 7) == 0;
        if (vec)
            ti_launch(sum_add_norm32_vec_kernel, dim3(n_rows), dim3(size >= 2048 ? 256 : 128), smem, stream, x, (const bf16*)d1, p1, n1, (size_t)s1,
                      (const bf16*)d2, p2, n2, (size_t)s2, (bf16*)h, (const bf16*)w_out, offset_out, eps_out, size);
        else
        ti_launch(sum_add_norm32_kernel<T>, dim3(n_rows), dim3(row_threads(size)), smem, stream, x, (const T*)d1, p1, n1, (size_t)s1, (const T*)d2, p2, n2,
                  (size_t)s2, (T*)h, (const T*)w_out, offset_out, eps_out, size);
    });
    return ti_check_launch("sum_add_norm32");
}
