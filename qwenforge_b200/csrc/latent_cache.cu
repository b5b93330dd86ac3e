// The two latents of a latent-attention mixer, from their fused down-projection:
//   down[t] = [ Dq h_t | Dkv h_t ]  (float32, q_rank + kv_rank columns)
//   a_t = down[t][:q_rank]  * rsqrt(mean(.^2) + eps) * q_norm      -> q_latent[t]    (what the query up-projection reads)
//   c_t = down[t][q_rank:]  * rsqrt(mean(.^2) + eps) * kv_norm     -> the cache row of the token's own position
// Both sums of squares and roots are float32. The key/value latent is the only thing the mixer keeps per position: it is
// written as the single "head" of a cache whose pages hold one plane, [pages][1][1][QF_PAGE][kv_rank]. With q_rank = 0
// there is no query latent and only the cache row is made. A padding entry (slot -1) writes no cache row; `latent_out`,
// if given, also receives c_t in token order (for whoever wants the step's latents without reading the cache).
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_cache_kernel(const float* __restrict__ down, int ld, int q_rank, int kv_rank, const T* __restrict__ q_norm,
                         const T* __restrict__ kv_norm, float eps, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                         const int* __restrict__ slots, T* __restrict__ q_latent, T* __restrict__ latent_out, KvSite<T> site,
                         int write_cache, int* err) {
    // the norm weights are nobody's output: a thread's first few are fetched before the wait for the kernel before this one
    grid_launch_dependents();
    constexpr int AHEAD = 4;
    float qw[AHEAD], kw[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
        const int c = threadIdx.x + u * 128;
        qw[u] = c < q_rank ? Num<T>::to_f(q_norm[c]) : 0.f;
        kw[u] = c < kv_rank ? Num<T>::to_f(kv_norm[c]) : 0.f;
    }
    grid_dependency_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* row = down + (size_t)t * ld;
    // where the latent goes: a chain of three dependent loads, started before the sums so that it runs under them
    T* cache_row = nullptr;
    const int slot = slots[tok_seq[t]];
    bool no_page = false;
    if (write_cache && slot >= 0) {
        cache_row = kv_row(site, slot, tok_pos[t], 0, 0);
        no_page = cache_row == nullptr;
    }
    if (q_rank > 0) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x) ss += row[c] * row[c];
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
        T* dst = q_latent + (size_t)t * q_rank;
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const int c = threadIdx.x + u * 128;
            if (c < q_rank) dst[c] = Num<T>::from_f(row[c] * inv * qw[u]);
        }
        for (int c = threadIdx.x + AHEAD * 128; c < q_rank; c += 128) dst[c] = Num<T>::from_f(row[c] * inv * Num<T>::to_f(q_norm[c]));
    }
    const float* kv = row + q_rank;
    float ss = 0.f;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) ss += kv[c] * kv[c];
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
    if (no_page && threadIdx.x == 0) atomicOr(err, QF_ERR_NO_PAGE);
    T* plain = latent_out ? latent_out + (size_t)t * kv_rank : nullptr;
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
        const int c = threadIdx.x + u * 128;
        if (c < kv_rank) {
            const T v = Num<T>::from_f(kv[c] * inv * kw[u]);
            if (cache_row) cache_row[c] = v;
            if (plain) plain[c] = v;
        }
    }
    for (int c = threadIdx.x + AHEAD * 128; c < kv_rank; c += 128) {
        const T v = Num<T>::from_f(kv[c] * inv * Num<T>::to_f(kv_norm[c]));
        if (cache_row) cache_row[c] = v;
        if (plain) plain[c] = v;
    }
}

template <typename T>
static int launch(const float* down, int ld, int q_rank, int kv_rank, const void* q_norm, const void* kv_norm, float eps,
                  const int* tok_seq, const int* tok_pos, const int* slots, void* q_latent, void* latent_out, void* base,
                  const int* table, long long page_elems, int table_stride, int write_cache, int n_tokens, int* err,
                  cudaStream_t stream) {
    KvSite<T> site{(T*)base, table, page_elems, table_stride, 1, kv_rank};
    return (int)launch_pdl(latent_norm_cache_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, down, ld, q_rank, kv_rank,
                           (const T*)q_norm, (const T*)kv_norm, eps, tok_seq, tok_pos, slots, (T*)q_latent, (T*)latent_out, site,
                           write_cache, err);
}

// down float32 [n_tokens][ld] (ld >= q_rank + kv_rank); the norm weights, q_latent [n_tokens][q_rank], latent_out
// [n_tokens][kv_rank] (may be null) and the cache share the activation dtype.
QF_EXPORT int qf_latent_norm_cache(int is_bf16, const float* down, int ld, int q_rank, int kv_rank, const void* q_norm,
                                   const void* kv_norm, float eps, const int* tok_seq, const int* tok_pos, const int* slots,
                                   void* q_latent, void* latent_out, void* base, const int* table, long long page_elems,
                                   int table_stride, int write_cache, int n_tokens, int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (kv_rank <= 0 || q_rank < 0 || ld < q_rank + kv_rank) return (int)cudaErrorInvalidValue;
    return is_bf16 ? launch<bf16>(down, ld, q_rank, kv_rank, q_norm, kv_norm, eps, tok_seq, tok_pos, slots, q_latent, latent_out,
                                  base, table, page_elems, table_stride, write_cache, n_tokens, err, stream)
                   : launch<float>(down, ld, q_rank, kv_rank, q_norm, kv_norm, eps, tok_seq, tok_pos, slots, q_latent, latent_out,
                                   base, table, page_elems, table_stride, write_cache, n_tokens, err, stream);
}
