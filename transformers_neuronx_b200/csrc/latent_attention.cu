// What lies around the paged attention kernels for an attention whose keys and values are expanded per head from one
// low-rank latent c per position, plus one rotated key part shared by all heads:
//     k_h = [W_uk,h c | r],  v_h = W_uv,h c,  score = scale * (q_plain,h . W_uk,h c + q_rot,h . r)
// Only c and r are kept per position, as ONE key/value head of `D` dims a position: the key row is [c | r | 0], the
// value row [c | 0].  The expansion moves to the queries' side: q'_h = [W_uk,h^T q_plain,h | q_rot,h | 0], whose product
// with the key row is the score above, and the attention's output per head, sum_j p_j c_j, goes through W_uv,h afterwards.
//
// tnx_latent_prep, one thread block per token at position p: from the output of the two down projections
//   (columns: rq of the queries' latent, rkv of the keys'/values' latent, dr of the rotated key part)
//     c_q = x / sqrt(mean(x^2) + eps) * wq  -> cq_out (the input of the queries' up projection)
//     c   = x / sqrt(mean(x^2) + eps) * wkv -> key row and value row
//     r turned by p (pairs (2i, 2i + 1) when interleaved, else (i, i + dr/2); angle p * inv_freq[i]) -> key row
// tnx_headwise_product: out[n, h, :n_out] = sum_k in[n, h, k] * W[h, k, :]  for every token n and head h, 32-bit sums
//   (W stored [heads, K, n_out]); a block takes one head and up to 8 tokens, so a head's matrix is read once per 8 tokens.
//   With rot_dims > 0 it also carries the head's rotated part over: in[n, h, K .. K + rot_dims) turned by the token's
//   position to out[n, h, n_out .. n_out + rot_dims), and zeroes the head's padding up to pad_to.  do_product = 0: only
//   that (the product was done elsewhere).
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ proj, int ld, int col0, const int* __restrict__ token_request,
                   const int* __restrict__ positions, const float* __restrict__ wq, const float* __restrict__ wkv,
                   float eps, const float* __restrict__ inv_freq, int interleaved, T* __restrict__ cq_out,
                   T* __restrict__ k_out, T* __restrict__ v_out, int rq, int rkv, int dr, int D) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    if (token_request[n] < 0) return;                  // a padded row of a captured step
    const float pos = (float)positions[n];
    const T* row = proj + (size_t)n * ld + col0;
    float sq = 0.f, sc = 0.f;
    for (int i = threadIdx.x; i < rq; i += blockDim.x) { const float x = to_float(row[i]); sq = fmaf(x, x, sq); }
    for (int i = threadIdx.x; i < rkv; i += blockDim.x) { const float x = to_float(row[rq + i]); sc = fmaf(x, x, sc); }
    const float rinv_q = 1.0f / sqrtf(block_sum(sq, scratch) / (float)rq + eps);
    const float rinv_c = 1.0f / sqrtf(block_sum(sc, scratch) / (float)rkv + eps);
    for (int i = threadIdx.x; i < rq; i += blockDim.x) {
        float x = to_float(row[i]) * rinv_q;
        if (wq) x *= wq[i];
        cq_out[(size_t)n * rq + i] = from_float<T>(x);
    }
    T* kd = k_out + (size_t)n * D;
    T* vd = v_out + (size_t)n * D;
    for (int i = threadIdx.x; i < rkv; i += blockDim.x) {
        float x = to_float(row[rq + i]) * rinv_c;
        if (wkv) x *= wkv[i];
        kd[i] = vd[i] = from_float<T>(x);
    }
    const T* rr = row + rq + rkv;
    for (int i = threadIdx.x; i < dr / 2; i += blockDim.x) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + dr / 2;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const float u = to_float(rr[ia]), v = to_float(rr[ib]);
        kd[rkv + ia] = from_float<T>(u * cs - v * sn);
        kd[rkv + ib] = from_float<T>(v * cs + u * sn);
    }
    for (int i = rkv + dr + threadIdx.x; i < D; i += blockDim.x) kd[i] = from_float<T>(0.f);
    for (int i = rkv + threadIdx.x; i < D; i += blockDim.x) vd[i] = from_float<T>(0.f);
}

constexpr int HP_TOKENS = 8;

template <typename T>
__global__ void __launch_bounds__(128)
headwise_product_kernel(const T* __restrict__ in, int in_ld, int in_head, const T* __restrict__ W, T* __restrict__ out,
                        int out_ld, int out_head, const int* __restrict__ token_request, const int* __restrict__ positions,
                        const float* __restrict__ inv_freq, int rot_dims, int interleaved, int pad_to, int do_product,
                        int N, int K, int n_out) {
    extern __shared__ float xs[];                      // [HP_TOKENS][K]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, n0 = blockIdx.y * HP_TOKENS;
    const int nt = min(HP_TOKENS, N - n0);
    if (do_product) {
        for (int e = threadIdx.x; e < nt * K; e += blockDim.x) {
            const int t = e / K, kk = e % K;
            xs[e] = token_request[n0 + t] < 0 ? 0.f : to_float(in[(size_t)(n0 + t) * in_ld + (size_t)h * in_head + kk]);
        }
        __syncthreads();
        const T* Wh = W + (size_t)h * K * n_out;
        for (int c = threadIdx.x; c < n_out; c += blockDim.x) {
            float acc[HP_TOKENS];
#pragma unroll
            for (int t = 0; t < HP_TOKENS; ++t) acc[t] = 0.f;
            for (int kk = 0; kk < K; ++kk) {
                const float w = to_float(Wh[(size_t)kk * n_out + c]);
#pragma unroll
                for (int t = 0; t < HP_TOKENS; ++t) acc[t] = fmaf(xs[t * K + kk], w, acc[t]);     // rows beyond nt: stale, unused
            }
#pragma unroll
            for (int t = 0; t < HP_TOKENS; ++t)
                if (t < nt && token_request[n0 + t] >= 0)
                    out[(size_t)(n0 + t) * out_ld + (size_t)h * out_head + c] = from_float<T>(acc[t]);
        }
    }
    if (pad_to <= n_out) return;
    const int half = rot_dims / 2, pad = pad_to - n_out - rot_dims;
    for (int e = threadIdx.x; e < nt * (half + pad); e += blockDim.x) {
        const int t = e / (half + pad), i = e % (half + pad), n = n0 + t;
        if (token_request[n] < 0) continue;
        T* dst = out + (size_t)n * out_ld + (size_t)h * out_head + n_out;
        if (i < half) {
            const T* src = in + (size_t)n * in_ld + (size_t)h * in_head + K;
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            float sn, cs;
            sincosf((float)positions[n] * inv_freq[i], &sn, &cs);
            const float u = to_float(src[ia]), v = to_float(src[ib]);
            dst[ia] = from_float<T>(u * cs - v * sn);
            dst[ib] = from_float<T>(v * cs + u * sn);
        } else {
            dst[rot_dims + i - half] = from_float<T>(0.f);
        }
    }
}

}  // namespace

TNX_EXPORT int tnx_latent_prep(const void* proj, int ld, int col0, const int* token_request, const int* positions,
                               const float* wq, const float* wkv, float eps, const float* inv_freq, int interleaved,
                               void* cq_out, void* k_out, void* v_out, int n_tokens, int rq, int rkv, int dr, int D,
                               int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rq <= 0 || rkv <= 0 || dr < 0 || dr % 2 || D < rkv + dr || (dr && !inv_freq)) return TNX_ERR_BAD_ARG;
    if (is_h16)
        return tnx_launch_in_order(latent_prep_kernel<h16>, dim3(n_tokens), dim3(128), 0, stream, (const h16*)proj, ld, col0,
                                   token_request, positions, wq, wkv, eps, inv_freq, interleaved, (h16*)cq_out,
                                   (h16*)k_out, (h16*)v_out, rq, rkv, dr, D);
    return tnx_launch_in_order(latent_prep_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, (const float*)proj, ld, col0,
                               token_request, positions, wq, wkv, eps, inv_freq, interleaved, (float*)cq_out,
                               (float*)k_out, (float*)v_out, rq, rkv, dr, D);
}

TNX_EXPORT int tnx_headwise_product(const void* in, int in_ld, int in_head, const void* W, void* out, int out_ld,
                                    int out_head, const int* token_request, const int* positions, const float* inv_freq,
                                    int rot_dims, int interleaved, int pad_to, int do_product, int n_tokens, int n_heads,
                                    int K, int n_out, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_heads <= 0 || K <= 0 || n_out <= 0 || rot_dims < 0 || rot_dims % 2 || (rot_dims && (!inv_freq || !positions)) ||
        (pad_to > n_out && pad_to < n_out + rot_dims) || (pad_to <= n_out && rot_dims) || (do_product && !W))
        return TNX_ERR_BAD_ARG;
    const size_t smem = do_product ? (size_t)HP_TOKENS * K * sizeof(float) : 0;
    if (smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const dim3 grid(n_heads, (n_tokens + HP_TOKENS - 1) / HP_TOKENS);
#define HPROD(T)                                                                                                         \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(headwise_product_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        return tnx_launch_in_order(headwise_product_kernel<T>, grid, dim3(128), smem, stream, (const T*)in, in_ld, in_head, \
                                   (const T*)W, (T*)out, out_ld, out_head, token_request, positions, inv_freq, rot_dims, \
                                   interleaved, pad_to, do_product, n_tokens, K, n_out);                                 \
    } while (0)
    if (is_h16) HPROD(h16);
    HPROD(float);
#undef HPROD
}
