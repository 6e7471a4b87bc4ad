// Inputs of latent attention: the two down-projected latents of a token, each RMS-normed in 32-bit with a plain
// weight; the query latent goes to a dense buffer, the key/value latent to the token's place in the paged pool
// (one "head" of kv_rank elements per position: pool[slot * kv_rank + i], slot = page * page_size + offset).
//
//   cq = T(a / rms(a) * wq),  a = row[0 : q_rank]
//   c  = T(b / rms(b) * wkv), b = row[q_rank : q_rank + kv_rank]
//
// With a rotated key part (rot > 0) the row has rot more elements after the two latents: one key part shared by all heads,
// not normed, rotated by the position's angles (cos_sin [positions, rot / 2, 2] float; pairs (2i, 2i + 1) or (i, i + rot / 2)) in
// 32-bit and written behind the latent in the same row of the pool, whose rows are pool_row >= kv_rank + rot long (zeros after).
// rotate_heads does the same rotation in place for a part of every head of a [n, heads, row] tensor (the queries' rotated part).
//
// The row is the fused down projection's output [n, q_rank + kv_rank] in T, or its 32-bit partial sums
// [s, n, q_rank + kv_rank] (a product cut over k), added in split order. One block per token.
#include "common.cuh"

#define LI_THREADS 128

template <typename T>
__global__ void latent_inputs_kernel(const T* rows, size_t row_stride, const float* partials, int n_partials, size_t partial_stride,
                                     T* __restrict__ cq, T* pool, const T* __restrict__ wq, const T* __restrict__ wkv, float eps,
                                     const int* slots, int q_rank, int kv_rank, int rot, const float* __restrict__ cos_sin, int interleaved,
                                     const int* positions, int pool_row, size_t in_row) {
    extern __shared__ float row[];             // [q_rank + kv_rank + rot]
    __shared__ float scratch[33];
    const int t = blockIdx.x, size = q_rank + kv_rank + rot, normed = q_rank + kv_rank;
    pdl_enter();
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < size; i += LI_THREADS) {
        float v;
        if (partials != nullptr) {
            const float* p = partials + (size_t)t * in_row + i;
            v = __ldcg(p);
            for (int s = 1; s < n_partials; ++s) v += __ldcg(p + (size_t)s * partial_stride);
        } else {
            v = to_f32(__ldcg(rows + (size_t)t * row_stride + i));
        }
        row[i] = v;
        if (i < q_rank) sq = fmaf(v, v, sq);
        else if (i < normed) sk = fmaf(v, v, sk);
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    const float iq = 1.0f / sqrtf(sq / (float)q_rank + eps), ik = 1.0f / sqrtf(sk / (float)kv_rank + eps);
    const size_t slot = (size_t)__ldcg(slots + t);
    for (int i = threadIdx.x; i < normed; i += LI_THREADS) {
        if (i < q_rank) cq[(size_t)t * q_rank + i] = from_f32<T>(row[i] * iq * to_f32(wq[i]));
        else pool[slot * pool_row + (i - q_rank)] = from_f32<T>(row[i] * ik * to_f32(wkv[i - q_rank]));
    }
    if (pool_row == kv_rank) return;
    const float* cs = rot > 0 ? cos_sin + (size_t)__ldcg(positions + t) * rot : nullptr;      // [rot / 2][2] = (cos, sin)
    const float* kr = row + normed;
    const int half = rot >> 1;
    for (int j = threadIdx.x; j < pool_row - kv_rank; j += LI_THREADS) {
        float v = 0.f;
        if (j < rot) {
            const int i = interleaved ? j >> 1 : (j < half ? j : j - half);
            const bool first = interleaved ? !(j & 1) : j < half;
            const float other = interleaved ? (first ? -kr[j + 1] : kr[j - 1]) : (first ? -kr[j + half] : kr[j - half]);
            v = kr[j] * cs[2 * i] + other * cs[2 * i + 1];
        }
        pool[slot * pool_row + kv_rank + j] = from_f32<T>(v);
    }
}

// x [n, heads, row] of T: elements [first, first + rot) of every head are rotated in place, a thread per pair, in 32-bit.
template <typename T>
__global__ void rotate_heads_kernel(T* x, const float* __restrict__ cos_sin, const int* positions, int heads, int row, int first, int rot,
                                    int interleaved, size_t pairs) {
    const int half = rot >> 1;
    pdl_enter();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < pairs; e += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(e % half);
        const size_t th = e / half;                    // token * heads + head
        const size_t t = th / heads;
        const float* cs = cos_sin + ((size_t)__ldcg(positions + t) * half + i) * 2;
        T* base = x + th * row + first;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        const float u = to_f32(base[a]), v = to_f32(base[b]);
        base[a] = from_f32<T>(u * cs[0] - v * cs[1]);
        base[b] = from_f32<T>(v * cs[0] + u * cs[1]);
    }
}

extern "C" int ti_rotate_heads(void* x, const float* cos_sin, const int* positions, int n, int heads, int row, int first, int rot, int interleaved,
                               int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(rot >= 2 && rot % 2 == 0 && first >= 0 && first + rot <= row && heads > 0, "rotate_heads: %d elements from %d in heads of %d", rot, first, row);
    const long long pairs = (long long)n * heads * (rot / 2);
    long long blocks = (pairs + 255) / 256;
    if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(rotate_heads_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)x, cos_sin, positions, heads, row, first,
                                        rot, interleaved, (size_t)pairs)));
    return ti_check_launch("rotate_heads");
}

extern "C" int ti_latent_inputs(const void* rows, long long row_stride, const float* partials, int n_partials, long long partial_stride,
                                void* cq, void* pool, const void* wq, const void* wkv, float eps, const int* slots, int n_tokens,
                                int q_rank, int kv_rank, int rot, const float* cos_sin, int interleaved, const int* positions, int pool_row,
                                long long in_row, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    TI_REQUIRE(q_rank > 0 && kv_rank > 0 && rot >= 0 && q_rank + kv_rank + rot <= 12000, "latent_inputs: ranks %d and %d, %d rotated", q_rank, kv_rank, rot);
    TI_REQUIRE((rows != nullptr) != (partials != nullptr), "latent_inputs: give rows or partial sums, not both");
    TI_REQUIRE(pool_row >= kv_rank + rot && in_row >= q_rank + kv_rank + rot, "latent_inputs: pool rows of %d for %d + %d", pool_row, kv_rank, rot);
    TI_REQUIRE(rot == 0 || (rot % 2 == 0 && cos_sin != nullptr && positions != nullptr), "latent_inputs: %d rotated elements need a table and positions", rot);
    const size_t smem = (size_t)(q_rank + kv_rank + rot) * sizeof(float);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(latent_inputs_kernel<T>, dim3(n_tokens), dim3(LI_THREADS), smem, stream, (const T*)rows,
                                        (size_t)row_stride, partials, n_partials, (size_t)partial_stride, (T*)cq, (T*)pool, (const T*)wq,
                                        (const T*)wkv, eps, slots, q_rank, kv_rank, rot, cos_sin, interleaved, positions, pool_row,
                                        (size_t)in_row)));
    return ti_check_launch("latent_inputs");
}
