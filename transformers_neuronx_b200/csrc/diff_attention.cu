// Differential attention around the paged attention kernels.  Every head holds two maps of queries and keys (dk dims
// each) over the same values (dv dims):
//     o = softmax(scale q1 k1^T) v - lambda softmax(scale q2 k2^T) v
// The two maps run as 2H query heads on the G key/value heads of ONE paged attention call, with rows of D dims
// (D >= 2 dk, D >= dv): a key row is [k1 | k2 | 0], the query of map 1 is [q1 | 0 | 0], that of map 2 is [0 | q2 | 0], so a
// score is the map's own product and a key/value head's pages are read once for both maps; a value row is [v | 0].
//
// tnx_diff_qkv_prep, per token, from one product's output `proj` (columns: queries [H][2][dk], then, unless G is 0, keys
//   [G][2][dk] and values [G][dv]):  every (head, map) of q and k divided by its root mean square (eps inside the root)
//   and multiplied by a weight vector of dk (one for all heads and maps; absent: none); queries then multiplied by
//   1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) at position p (temp_every 0: not); all in 32-bit, written in the
//   activation type in the layout above (query head index 2 h + map).
// tnx_diff_combine, per (token, head), from the attention's output [N, 2H, D]:
//   o = a1 - lambda a2;  o / sqrt(mean(o^2) + eps) * out_mult * sigmoid(gate logit of the head) * out_scale
//   written to the output projection's input [N, H * dv] in the activation type.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
diff_qkv_prep_kernel(const T* __restrict__ proj, int ld, int col0, const int* __restrict__ token_request,
                     const int* __restrict__ positions, const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                     float eps, float temp_coef, int temp_every, T* __restrict__ q_out, T* __restrict__ k_out,
                     T* __restrict__ v_out, int H, int G, int dk, int dv, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    if (token_request[n] < 0) return;                        // a padded row of a captured step
    const T* row = proj + (size_t)n * ld + col0;
    float temp = 1.f;
    if (temp_every > 0) temp = 1.f + temp_coef * logf((float)((positions[n] + 1) / temp_every) + 1.f);
    const int q_units = 2 * H, k_units = 2 * G;
    for (int u = blockIdx.y * warps + warp; u < q_units + k_units + G; u += gridDim.y * warps) {
        if (u < q_units + k_units) {
            const bool is_q = u < q_units;
            const int unit = is_q ? u : u - q_units;         // (head, map) = (unit / 2, unit % 2)
            const T* src = row + (is_q ? 0 : q_units * dk) + unit * dk;
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) { const float x = to_float(src[i]); ss = fmaf(x, x, ss); }
            float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
            if (is_q) rinv *= temp;
            const float* w = is_q ? q_norm : k_norm;
            // a query's row holds its own map only; a key's row holds both maps side by side
            T* dst = is_q ? q_out + ((size_t)n * q_units + unit) * D : k_out + ((size_t)n * G + unit / 2) * D;
            const int at = (unit & 1) * dk;
            for (int i = lane; i < dk; i += 32) dst[at + i] = from_float<T>(to_float(src[i]) * rinv * (w ? w[i] : 1.f));
            if (is_q) {
                for (int i = lane; i < D; i += 32)
                    if (i < at || i >= at + dk) dst[i] = from_float<T>(0.f);
            } else if (unit & 1) {
                for (int i = 2 * dk + lane; i < D; i += 32) dst[i] = from_float<T>(0.f);
            }
        } else {
            const int g = u - q_units - k_units;
            const T* src = row + (q_units + k_units) * dk + g * dv;
            T* dst = v_out + ((size_t)n * G + g) * D;
            for (int i = lane; i < D; i += 32) dst[i] = i < dv ? src[i] : from_float<T>(0.f);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T* __restrict__ att, const T* __restrict__ gate, int gate_ld, const int* __restrict__ token_request,
                    float lambda, float eps, float out_mult, float out_scale, T* __restrict__ out, int out_ld, int n_tokens,
                    int H, int dv, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (pair >= (long long)n_tokens * H) return;
    const int n = (int)(pair / H), h = (int)(pair % H);
    if (token_request[n] < 0) return;
    const T* a1 = att + ((size_t)n * 2 * H + 2 * h) * D;
    const T* a2 = a1 + D;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) {
        const float o = to_float(a1[i]) - lambda * to_float(a2[i]);
        ss = fmaf(o, o, ss);
    }
    float mult = out_mult * out_scale / sqrtf(warp_sum(ss) / (float)dv + eps);
    if (gate) mult *= 1.f / (1.f + expf(-to_float(gate[(size_t)n * gate_ld + h])));
    T* dst = out + (size_t)n * out_ld + (size_t)h * dv;
    for (int i = lane; i < dv; i += 32) dst[i] = from_float<T>((to_float(a1[i]) - lambda * to_float(a2[i])) * mult);
}

}  // namespace

TNX_EXPORT int tnx_diff_qkv_prep(const void* proj, int ld, int col0, const int* token_request, const int* positions,
                                 const float* q_norm, const float* k_norm, float eps, float temp_coef, int temp_every,
                                 void* q_out, void* k_out, void* v_out, int N, int H, int G, int dk, int dv, int D,
                                 int is_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || G < 0 || dk <= 0 || dv <= 0 || D < 2 * dk || D < dv || temp_every < 0) return TNX_ERR_BAD_ARG;
    const int units = 2 * H + 3 * G;
    // a prompt's tokens: one block a token; the few tokens of a decode step: a token's units over several blocks
    const int ny = N >= 256 ? 1 : (units + 3) / 4 < 8 ? (units + 3) / 4 : 8;
    const dim3 grid(N, ny);
    if (is_h16)
        return tnx_launch_in_order(diff_qkv_prep_kernel<h16>, grid, dim3(128), 0, stream, (const h16*)proj, ld, col0,
                                   token_request, positions, q_norm, k_norm, eps, temp_coef, temp_every, (h16*)q_out,
                                   (h16*)k_out, (h16*)v_out, H, G, dk, dv, D);
    return tnx_launch_in_order(diff_qkv_prep_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, ld, col0,
                               token_request, positions, q_norm, k_norm, eps, temp_coef, temp_every, (float*)q_out,
                               (float*)k_out, (float*)v_out, H, G, dk, dv, D);
}

TNX_EXPORT int tnx_diff_combine(const void* att, const void* gate, int gate_ld, const int* token_request, float lambda,
                                float eps, float out_mult, float out_scale, void* out, int out_ld, int N, int H, int dv,
                                int D, int is_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || dv <= 0 || D < dv || out_ld < H * dv) return TNX_ERR_BAD_ARG;
    const int warps = 4;
    const long long pairs = (long long)N * H;
    const int blocks = (int)((pairs + warps - 1) / warps);
    if (is_h16)
        return tnx_launch_in_order(diff_combine_kernel<h16>, dim3(blocks), dim3(warps * 32), 0, stream, (const h16*)att,
                                   (const h16*)gate, gate_ld, token_request, lambda, eps, out_mult, out_scale, (h16*)out,
                                   out_ld, N, H, dv, D);
    return tnx_launch_in_order(diff_combine_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, (const float*)att,
                               (const float*)gate, gate_ld, token_request, lambda, eps, out_mult, out_scale, (float*)out,
                               out_ld, N, H, dv, D);
}
