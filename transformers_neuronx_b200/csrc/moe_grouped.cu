// Routed experts on the tensor cores: the (token, chosen expert) pairs are sorted by expert into a layout in which every
// expert's rows begin at a multiple of the tile (128 rows where experts get many rows; 16, 32 or 64 where they get few),
// so that each tile belongs to one expert and the two products of an expert run as grouped tensor-core products
// (gemm_tc.cu: tnx_gemm_tc_grouped, tnx_gemm_tc_grouped_few).  The kernels of this file are what lies around those products:
//
//   moe_plan_kernel      one block: counts per expert, every expert's first row, the expert of every tile (-1 beyond
//                        the last used tile), and the row of every pair.  Which row of its expert's segment a pair
//                        gets depends on the order in which threads arrive; a row's result does not depend on where it sits
//   moe_gather_kernel    x[row(pair)] = weight * h[token]  (or h[token] when the weight multiplies the output), 16-bit
//   moe_act_kernel       y = g * sigmoid(alpha g) * (u + up_shift), g and u clamped, from the gate/up product's output
//                        (moe_act_relu2_kernel: y = relu(u)^2 for experts without a gate)
//   moe_combine_kernel   out[token] (+)= sum over the token's pairs, in the order of the choice, of the down product's rows
//
// Nothing is read on the host: the sizes of the buffers follow from the numbers of tokens and experts alone (at most
// pairs / tile + experts tiles), so a step can be captured in a CUDA graph.
#include "common.cuh"

namespace {
constexpr int MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int max_tiles, int TILE, int* __restrict__ group_of_tile,
                int* __restrict__ row_of_pair) {
    __shared__ int count[MAX_EXPERTS], first[MAX_EXPERTS], cursor[MAX_EXPERTS];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            first[e] = tile * TILE;
            const int t = (count[e] + TILE - 1) / TILE;
            for (int j = 0; j < t && tile + j < max_tiles; ++j) group_of_tile[tile + j] = e;
            tile += t;
        }
        for (; tile < max_tiles; ++tile) group_of_tile[tile] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = ids[i];
        row_of_pair[i] = e >= 0 ? first[e] + atomicAdd(&cursor[e], 1) : -1;
    }
}

__global__ void __launch_bounds__(128)
moe_gather_kernel(const h16* __restrict__ h, int ld, const float* __restrict__ weights, const int* __restrict__ row_of_pair,
                  h16* __restrict__ x, int W, int top, int weight_on_input) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x, row = row_of_pair[pair];
    if (row < 0) return;
    const float wt = weight_on_input ? weights[pair] : 1.f;
    const h16* src = h + (size_t)(pair / top) * ld;
    h16* dst = x + (size_t)row * W;
    if (W % 8 == 0 && ld % 8 == 0 && !(((uintptr_t)h | (uintptr_t)x) & 15)) {
        for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
            uint4 raw = *(const uint4*)(src + c);
            h16x2* v = (h16x2*)&raw;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = h16x2_to_float2(v[i]);
                v[i] = floats_to_h16x2(f.x * wt, f.y * wt);
            }
            *(uint4*)(dst + c) = raw;
        }
    } else {
        for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = float_to_h16(h16_to_float(src[c]) * wt);
    }
}

__global__ void __launch_bounds__(256)
moe_act_kernel(const h16* __restrict__ gu, h16* __restrict__ y, const int* __restrict__ group_of_tile, int TILE, int F,
               float gate_max, float up_min, float up_max, float alpha, float up_shift) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    if (group_of_tile[row / TILE] < 0) return;
    const h16* g = gu + (size_t)row * 2 * F;
    const h16* u = g + F;
    for (int c = threadIdx.x * 2; c < F; c += blockDim.x * 2) {
        if (c + 1 < F && F % 2 == 0) {
            const float2 gf = h16x2_to_float2(*(const h16x2*)(g + c)), uf = h16x2_to_float2(*(const h16x2*)(u + c));
            const float g0 = fminf(gf.x, gate_max), g1 = fminf(gf.y, gate_max);
            const float u0 = fminf(fmaxf(uf.x, up_min), up_max), u1 = fminf(fmaxf(uf.y, up_min), up_max);
            *(h16x2*)(y + (size_t)row * F + c) = floats_to_h16x2(g0 / (1.f + expf(-alpha * g0)) * (u0 + up_shift),
                                                                 g1 / (1.f + expf(-alpha * g1)) * (u1 + up_shift));
        } else {
            for (int i = c; i < min(c + 2, F); ++i) {
                const float g0 = fminf(h16_to_float(g[i]), gate_max);
                const float u0 = fminf(fmaxf(h16_to_float(u[i]), up_min), up_max);
                y[(size_t)row * F + i] = float_to_h16(g0 / (1.f + expf(-alpha * g0)) * (u0 + up_shift));
            }
        }
    }
}

// Experts without a gate: y = relu(u)^2 from the up product's output [rows, F].
__global__ void __launch_bounds__(256)
moe_act_relu2_kernel(const h16* __restrict__ u, h16* __restrict__ y, const int* __restrict__ group_of_tile, int TILE, int F) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    if (group_of_tile[row / TILE] < 0) return;
    const h16* src = u + (size_t)row * F;
    h16* dst = y + (size_t)row * F;
    if (F % 2 == 0) {
        for (int c = threadIdx.x * 2; c < F; c += blockDim.x * 2) {
            const float2 f = h16x2_to_float2(*(const h16x2*)(src + c));
            const float a = fmaxf(f.x, 0.f), b = fmaxf(f.y, 0.f);
            *(h16x2*)(dst + c) = floats_to_h16x2(a * a, b * b);
        }
    } else {
        for (int c = threadIdx.x; c < F; c += blockDim.x) {
            const float a = fmaxf(h16_to_float(src[c]), 0.f);
            dst[c] = float_to_h16(a * a);
        }
    }
}

__global__ void __launch_bounds__(128)
moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ row_of_pair, const float* __restrict__ weights,
                   float* out, int W, int top, int accumulate, int weight_on_input) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    if (row_of_pair[(size_t)n * top] < 0) return;                 // a padded row of a captured step
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; ++j) {
            const float v = rows[(size_t)row_of_pair[(size_t)n * top + j] * W + c];
            s += weight_on_input ? v : v * weights[(size_t)n * top + j];
        }
        float* dst = out + (size_t)n * W + c;
        *dst = accumulate ? *dst + s : s;
    }
}
}  // namespace

// The most tiles that n_pairs pairs spread over n_experts experts can take.
TNX_EXPORT int tnx_moe_grouped_max_tiles(int n_pairs, int n_experts, int tile) {
    return n_pairs / tile + (n_pairs < n_experts ? n_pairs : n_experts);
}

TNX_EXPORT int tnx_moe_plan(const int* ids, int n_pairs, int n_experts, int max_tiles, int tile, int* group_of_tile,
                            int* row_of_pair, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts <= 0 || n_experts > MAX_EXPERTS || tile <= 0 || max_tiles < tnx_moe_grouped_max_tiles(n_pairs, n_experts, tile))
        return TNX_ERR_BAD_ARG;
    return tnx_launch_in_order(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, ids, n_pairs, n_experts, max_tiles, tile,
                               group_of_tile, row_of_pair);
}

TNX_EXPORT int tnx_moe_gather(const void* h, int ld, const float* weights, const int* row_of_pair, void* x, int n_pairs, int W,
                              int top, int weight_on_input, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    return tnx_launch_in_order(moe_gather_kernel, dim3(n_pairs), dim3(128), 0, stream, (const h16*)h, ld, weights, row_of_pair,
                               (h16*)x, W, top, weight_on_input);
}

TNX_EXPORT int tnx_moe_act(const void* gu, void* y, const int* group_of_tile, int tile, int rows, int F, float gate_max,
                           float up_min, float up_max, float alpha, float up_shift, int form, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (form == 1)
        return tnx_launch_in_order(moe_act_relu2_kernel, dim3(rows), dim3(F >= 512 ? 256 : 128), 0, stream, (const h16*)gu,
                                   (h16*)y, group_of_tile, tile, F);
    return tnx_launch_in_order(moe_act_kernel, dim3(rows), dim3(F >= 512 ? 256 : 128), 0, stream, (const h16*)gu, (h16*)y,
                               group_of_tile, tile, F, gate_max, up_min, up_max, alpha, up_shift);
}

TNX_EXPORT int tnx_moe_combine(const float* rows, const int* row_of_pair, const float* weights, float* out, int N, int W, int top,
                               int accumulate, int weight_on_input, cudaStream_t stream) {
    if (N <= 0) return 0;
    // few tokens: a slice of the width a block, so that the loads of a row are asked for together
    return tnx_launch_in_order(moe_combine_kernel, dim3(N, N >= 256 ? 1 : (W + 511) / 512), dim3(128), 0, stream, rows, row_of_pair, weights, out, W, top,
                               accumulate, weight_on_input);
}
