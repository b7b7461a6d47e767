// A feed-forward of routed experts.
//
//   z = W_r h                                  router logits, 32-bit sums
//   s = sigmoid(z) (or softmax(z))             scores; the `top` largest choose the token's experts
//   w_j = s[e_j] (optionally divided by their sum)
//   expert e on input x:  g = W_gate x, u = W_up x (both clamped where the part gives limits),
//                         y = g * sigmoid(alpha g) * (u + up_shift),  result W_down y
//   out = sum_j expert_{e_j}(w_j h)   (weight on the input)    or    sum_j w_j expert_{e_j}(h)   (on the output)
//   an expert without a gate (form 1):  y = relu(W_up x)^2,  result W_down y
//   routing options (sigmoid scores): a correction per expert added to the scores for the CHOICE only; experts in equal
//   groups of neighbours, a group scored by the sum of its group_top largest choice scores, only the keep_groups best
//   groups' experts open to the choice; weights w_j / (sum_j w_j + renorm_eps) * weight_scale
//
// Kernels of this file (T: the activations' type, TW: the stored type of the experts' matrices):
//   moe_router_kernel      a block a token: logits, scores, the top experts and their weights
//   moe_gate_up_kernel     a block per (expert, slice of the inner width): the inputs of the tokens that chose the expert
//                          in shared memory (four at a time), a warp per inner feature, 16-byte loads along the rows
//   moe_down_kernel        a block per (expert, slice of the width): the same for the down product, one 32-bit row per pair
//   moe_sum_kernel         adds a token's pairs up in the order of the choice and writes or adds the 32-bit result
// They stream a chosen expert's matrices once for every four tokens that chose it, through the multiply-add units: the
// form of the 32-bit engine and of sizes the tensor-core product refuses.  A 16-bit engine takes the grouped tensor-core
// products of moe_grouped.cu at every number of tokens (and this file's router).
#include "common.cuh"

namespace {
constexpr int MAX_TOP = 16;
constexpr int MAX_EXPERTS = 1024;

// 8 elements of a matrix as they are loaded (converted when they are used, so that several loads can be in flight).
template <typename TW> struct Raw8;
template <> struct Raw8<h16> {
    uint4 raw;
    __device__ __forceinline__ void load(const h16* p) { raw = *(const uint4*)p; }
    __device__ __forceinline__ void get(float (&v)[8]) const {
        const h16x2* h = (const h16x2*)&raw;
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = h16x2_to_float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static constexpr int AHEAD = 4;
};
template <> struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = *(const float4*)p; b = *(const float4*)(p + 4); }
    __device__ __forceinline__ void get(float (&v)[8]) const {
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static constexpr int AHEAD = 2;
};

// <w, x> over K elements by one warp; every lane gets the sum.  The order of the additions depends on K alone.  A lane
// asks for AHEAD pieces of 16 bytes before it uses the first.
template <typename TW>
__device__ __forceinline__ float warp_dot(const TW* __restrict__ w, const float* x, int K, int lane, bool vec) {
    constexpr int U = Raw8<TW>::AHEAD;
    float s = 0.f;
    if (vec) {
        for (int c = lane * 8; c < K; c += 256 * U) {
            Raw8<TW> a[U];
#pragma unroll
            for (int u = 0; u < U; ++u) if (c + 256 * u < K) a[u].load(w + c + 256 * u);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (c + 256 * u < K) {
                    float af[8];
                    a[u].get(af);
#pragma unroll
                    for (int i = 0; i < 8; ++i) s = fmaf(af[i], x[c + 256 * u + i], s);
                }
            }
        }
    } else {
        for (int c = lane; c < K; c += 32) s = fmaf(to_float(w[c]), x[c], s);
    }
    return warp_sum(s);
}

struct RouterOptions {
    const float* correction;     // [E] or null
    int n_groups, keep_groups, group_top;
    float renorm_eps, weight_scale;
};

template <typename T, typename TW>
__global__ void __launch_bounds__(128)
moe_router_kernel(const T* __restrict__ h, int ld, const TW* __restrict__ wr, const int* __restrict__ token_request,
                  int* __restrict__ ids, float* __restrict__ weights, int W, int E, int top, int softmax_scores,
                  int renormalize, RouterOptions ro) {
    extern __shared__ __align__(16) float sm[];            // [W] the row, [E] the logits (or choice scores), [E] the scores, [E] groups
    float* x = sm;
    float* z = sm + ((W + 3) & ~3);
    float* sc = z + E;
    float* gscore = sc + E;
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (token_request[n] < 0) {                              // a padded row of a captured step: no expert
        if (threadIdx.x < top) { ids[(size_t)n * top + threadIdx.x] = -1; weights[(size_t)n * top + threadIdx.x] = 0.f; }
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) x[c] = to_float(h[(size_t)n * ld + c]);
    __syncthreads();
    const bool vec = W % 8 == 0 && ((uintptr_t)wr % 16) == 0;
    for (int e = warp; e < E; e += 4) {
        const float s = warp_dot<TW>(wr + (size_t)e * W, x, W, lane, vec);
        if (lane == 0) z[e] = s;
    }
    __syncthreads();
    if (warp != 0) return;
    // The choice is made on the logits: both scores grow with them, and a sigmoid that has run out of bits near 1
    // would tie experts that their logits still tell apart.  With a correction or groups the choice is made on
    // choice score = sigmoid + correction, as the design says, and the weight is the uncorrected sigmoid.
    const bool corrected = ro.correction != nullptr || ro.n_groups > 1;
    if (corrected) {
        for (int e = lane; e < E; e += 32) {
            const float s0 = 1.f / (1.f + expf(-z[e]));
            sc[e] = s0;
            z[e] = s0 + (ro.correction ? ro.correction[e] : 0.f);
        }
        __syncwarp();
        if (ro.n_groups > 1) {
            const int size = E / ro.n_groups;
            for (int g = lane; g < ro.n_groups; g += 32) {          // the sum of the group's largest choice scores
                float total = 0.f;
                unsigned long long taken = 0ull;                     // group_top is small: a pass per pick
                for (int j = 0; j < ro.group_top && j < size; ++j) {
                    float best = -INFINITY;
                    int arg = -1;
                    for (int i = 0; i < size; ++i) {
                        if (i < 64 && (taken >> i & 1ull)) continue;
                        const float v = z[g * size + i];
                        if (arg < 0 || v > best) { best = v; arg = i; }
                    }
                    if (arg >= 0 && arg < 64) taken |= 1ull << arg;
                    total += best;
                }
                gscore[g] = total;
            }
            __syncwarp();
            // the keep_groups best groups stay (of equal ones the lowest index); the others' experts cannot be chosen
            for (int j = 0; j < ro.keep_groups; ++j) {
                float best = -INFINITY;
                int arg = 0x7fffffff;
                for (int g = lane; g < ro.n_groups; g += 32) {
                    const float v = gscore[g];
                    if (v == v && (v > best || arg == 0x7fffffff) && v != INFINITY) { best = v; arg = g; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                    if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
                }
                if (lane == 0 && arg != 0x7fffffff) gscore[arg] = INFINITY;      // kept
                __syncwarp();
            }
            for (int e = lane; e < E; e += 32)
                if (gscore[e / size] != INFINITY) z[e] = -INFINITY;
            __syncwarp();
        }
    }
    float mx = -INFINITY, sum = 0.f;
    if (softmax_scores) {
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
        sum = warp_sum(sum);
    }
    float chosen_w[MAX_TOP];
    int chosen[MAX_TOP];
    float total = 0.f;
    for (int j = 0; j < top; ++j) {                         // the largest logit left; of equal ones the lowest index
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        chosen[j] = arg;
        chosen_w[j] = corrected ? sc[arg] : (softmax_scores ? expf(best - mx) / sum : 1.f / (1.f + expf(-best)));
        total += chosen_w[j];
        if (lane == 0) z[arg] = -INFINITY;
        __syncwarp();
    }
    if (lane == 0)
        for (int j = 0; j < top; ++j) {
            ids[(size_t)n * top + j] = chosen[j];
            weights[(size_t)n * top + j] = (renormalize ? chosen_w[j] / (total + ro.renorm_eps) : chosen_w[j]) * ro.weight_scale;
        }
}

struct ExpertMath {
    float gate_max, up_min, up_max;     // clamps (infinite: none)
    float alpha, up_shift;              // y = g * sigmoid(alpha g) * (u + up_shift)
    int weight_on_input;
    int form;                           // 0: gated as above;  1: no gate, y = relu(u)^2
};

__device__ __forceinline__ float expert_act(float g, float u, const ExpertMath& m) {
    if (m.form == 1) { const float r = fmaxf(g, 0.f); return r * r; }      // without a gate the one product arrives as g
    g = fminf(g, m.gate_max);
    u = fminf(fmaxf(u, m.up_min), m.up_max);
    return g / (1.f + expf(-m.alpha * g)) * (u + m.up_shift);
}

// The pairs (token, choice) that chose expert e, in ascending order, gathered by warp 0 into `list`; returns their number
// to every thread.  (A step of few tokens: a few hundred pairs at most.)
__device__ __forceinline__ int pairs_of_expert(const int* __restrict__ ids, int n_pairs, int e, int* list, int* count_s) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int count = 0;
        for (int base = 0; base < n_pairs; base += 32) {
            const int i = base + lane;
            const bool mine = i < n_pairs && ids[i] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) list[count + __popc(mask & ((1u << lane) - 1u))] = i;
            count += __popc(mask);
        }
        if (lane == 0) *count_s = count;
    }
    __syncthreads();
    return *count_s;
}

template <typename T> struct Load8;
template <> struct Load8<h16> {
    static __device__ __forceinline__ void get(const h16* p, float (&v)[8]) {
        const uint4 raw = *(const uint4*)p;
        const h16x2* h = (const h16x2*)&raw;
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = h16x2_to_float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
};
template <> struct Load8<float> {
    static __device__ __forceinline__ void get(const float* p, float (&v)[8]) {
        const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};

constexpr int MT = 4;          // rows of one expert that share one pass over its matrices

// One pass over the rows `w0` and (when given) `w1` of length K for up to MT staged rows xs[r][K]: acc0[r] = <w0, xs[r]>.
// A lane asks for AHEAD pieces of 16 bytes of every row before it uses the first: with a row or two of tokens the
// kernel does little arithmetic per byte, and the bytes in flight are what the memory's rate depends on.
// R: how many rows are staged, as a constant (a count that is only known when the kernel runs made the compiler issue
// all rows' instructions under predicates: with eight rows 190 instructions per 16 bytes of weights where two rows need 50).
template <typename T, typename TW, bool TWO, int R>
__device__ __forceinline__ void rows_dot_n(const TW* __restrict__ w0, const TW* __restrict__ w1, const T* xs, int K,
                                           int lane, bool vec, float (&acc0)[MT], float (&acc1)[MT]) {
    constexpr int U = Raw8<TW>::AHEAD;
    constexpr int rows = R;
#pragma unroll
    for (int r = 0; r < MT; ++r) { acc0[r] = 0.f; acc1[r] = 0.f; }
    if (vec) {
        for (int c = lane * 8; c < K; c += 256 * U) {
            Raw8<TW> a[U], b[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int cc = c + 256 * u;
                if (cc < K) { a[u].load(w0 + cc); if (TWO) b[u].load(w1 + cc); }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int cc = c + 256 * u;
                if (cc < K) {
                    float af[8], bf[8], x[8];
                    a[u].get(af);
                    if (TWO) b[u].get(bf);
#pragma unroll
                    for (int r = 0; r < MT; ++r) {
                        if (r < rows) {
                            Load8<T>::get(xs + (size_t)r * K + cc, x);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                acc0[r] = fmaf(af[i], x[i], acc0[r]);
                                if (TWO) acc1[r] = fmaf(bf[i], x[i], acc1[r]);
                            }
                        }
                    }
                }
            }
        }
    } else {
        for (int c = lane; c < K; c += 32) {
            const float a = to_float(w0[c]), b = TWO ? to_float(w1[c]) : 0.f;
#pragma unroll
            for (int r = 0; r < MT; ++r) {
                if (r < rows) {
                    const float x = to_float(xs[(size_t)r * K + c]);
                    acc0[r] = fmaf(a, x, acc0[r]);
                    if (TWO) acc1[r] = fmaf(b, x, acc1[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < MT; ++r) {
        if (r < rows) {
            acc0[r] = warp_sum(acc0[r]);
            if (TWO) acc1[r] = warp_sum(acc1[r]);
        }
    }
}
template <typename T, typename TW, bool TWO>
__device__ __forceinline__ void rows_dot(const TW* __restrict__ w0, const TW* __restrict__ w1, const T* xs, int K, int rows,
                                         int lane, bool vec, float (&acc0)[MT], float (&acc1)[MT]) {
    switch (rows) {
        case 1: rows_dot_n<T, TW, TWO, 1>(w0, w1, xs, K, lane, vec, acc0, acc1); break;
        case 2: rows_dot_n<T, TW, TWO, 2>(w0, w1, xs, K, lane, vec, acc0, acc1); break;
        case 3: rows_dot_n<T, TW, TWO, 3>(w0, w1, xs, K, lane, vec, acc0, acc1); break;
        default: rows_dot_n<T, TW, TWO, MT>(w0, w1, xs, K, lane, vec, acc0, acc1); break;
    }
}

// gate_up: [E, 2F, W] (an expert's gate rows, then its up rows); y: [N * top, F] in the activations' type.
// A block per (expert, slice of the inner width): the expert's rows are streamed once for all the tokens that chose it
// (MT of them at a time, their inputs staged in shared memory in the activations' type); an expert nobody chose costs
// one look at the choices.
template <typename T, typename TW>
__global__ void __launch_bounds__(128, 4)
moe_gate_up_kernel(const T* __restrict__ h, int ld, const TW* __restrict__ gate_up, const int* __restrict__ ids,
                   const float* __restrict__ weights, T* __restrict__ y, int W, int F, int top, int n_pairs, int per_block,
                   ExpertMath m) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* xs = (T*)smem_raw;                                  // [MT][W]
    int* list = (int*)(smem_raw + (((size_t)MT * W * sizeof(T) + 15) & ~(size_t)15));
    __shared__ int count_s;
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int count = pairs_of_expert(ids, n_pairs, e, list, &count_s);
    if (count == 0) return;
    const bool gated = m.form == 0;                      // without a gate: [E, F, W], the up rows alone
    const TW* wg = gate_up + (size_t)e * (gated ? 2 : 1) * F * W;
    const TW* wu = wg + (size_t)F * W;
    const bool vec = W % 8 == 0 && ((uintptr_t)gate_up % 16) == 0;
    const int f_end = min(F, (blockIdx.y + 1) * per_block);
    for (int c0 = 0; c0 < count; c0 += MT) {
        const int rows = min(MT, count - c0);
        __syncthreads();
        for (int r = 0; r < rows; ++r) {
            const int pair = list[c0 + r];
            const float wt = m.weight_on_input ? weights[pair] : 1.f;
            const T* src = h + (size_t)(pair / top) * ld;
            T* dst = xs + (size_t)r * W;
            if (vec && ld % 8 == 0 && ((uintptr_t)h % 16) == 0) {
                for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
                    float v[8];
                    Load8<T>::get(src + c, v);
#pragma unroll
                    for (int i = 0; i < 8; ++i) dst[c + i] = from_float<T>(wt * v[i]);
                }
            } else {
                for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = from_float<T>(wt * to_float(src[c]));
            }
        }
        __syncthreads();
        for (int f = blockIdx.y * per_block + warp; f < f_end; f += 4) {
            float g[MT], u[MT];
            if (gated) rows_dot<T, TW, true>(wg + (size_t)f * W, wu + (size_t)f * W, xs, W, rows, lane, vec, g, u);
            else rows_dot<T, TW, false>(wg + (size_t)f * W, nullptr, xs, W, rows, lane, vec, g, u);
#pragma unroll
            for (int r = 0; r < MT; ++r)
                if (r < rows && lane == r) y[(size_t)list[c0 + r] * F + f] = from_float<T>(expert_act(g[r], u[r], m));
        }
    }
}

// down: [E, W, F]; per_pair: 32-bit [N * top, W], the chosen expert's result for every pair (moe_sum_kernel adds a
// token's pairs up).  A block per (expert, slice of the width), as above.
template <typename T, typename TW>
__global__ void __launch_bounds__(128, 4)
moe_down_kernel(const T* __restrict__ y, const TW* __restrict__ down, const int* __restrict__ ids, float* __restrict__ per_pair,
                int W, int F, int n_pairs, int per_block) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* ys = (T*)smem_raw;                                  // [MT][F]
    int* list = (int*)(smem_raw + (((size_t)MT * F * sizeof(T) + 15) & ~(size_t)15));
    __shared__ int count_s;
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int count = pairs_of_expert(ids, n_pairs, e, list, &count_s);
    if (count == 0) return;
    const bool vec = F % 8 == 0 && ((uintptr_t)down % 16) == 0 && ((uintptr_t)y % 16) == 0;
    const int o_end = min(W, (blockIdx.y + 1) * per_block);
    for (int c0 = 0; c0 < count; c0 += MT) {
        const int rows = min(MT, count - c0);
        __syncthreads();
        for (int i = threadIdx.x; i < rows * F; i += blockDim.x) {
            const int r = i / F, c = i - r * F;
            ys[(size_t)r * F + c] = y[(size_t)list[c0 + r] * F + c];
        }
        __syncthreads();
        for (int o = blockIdx.y * per_block + warp; o < o_end; o += 4) {
            float s[MT], unused[MT];
            rows_dot<T, TW, false>(down + ((size_t)e * W + o) * F, nullptr, ys, F, rows, lane, vec, s, unused);
#pragma unroll
            for (int r = 0; r < MT; ++r)
                if (r < rows && lane == r) per_pair[(size_t)list[c0 + r] * W + o] = s[r];
        }
    }
}

// out[n] (+)= sum over the token's choices, in their order, of per_pair (times the choice's weight where it multiplies
// the expert's output).
__global__ void __launch_bounds__(128)
moe_sum_kernel(const float* __restrict__ per_pair, const int* __restrict__ ids, const float* __restrict__ weights, float* out,
               int W, int top, int accumulate, int weight_on_input) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    if (ids[(size_t)n * top] < 0) return;                   // a padded row of a captured step
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; ++j) {
            const float v = per_pair[((size_t)n * top + j) * W + c];
            s += weight_on_input ? v : v * weights[(size_t)n * top + j];
        }
        float* dst = out + (size_t)n * W + c;
        *dst = accumulate ? *dst + s : s;
    }
}
}  // namespace

TNX_EXPORT int tnx_moe_route(const void* h, int ld, const void* router, const int* token_request, int* ids, float* weights,
                             int N, int W, int E, int top, int softmax_scores, int renormalize, int h_h16, int w_h16,
                             const float* correction, int n_groups, int keep_groups, int group_top, float renorm_eps,
                             float weight_scale, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (W <= 0 || E <= 0 || E > MAX_EXPERTS || top <= 0 || top > MAX_TOP || top > E) return TNX_ERR_UNSUPPORTED;
    if (n_groups < 1 || E % n_groups || keep_groups < 1 || keep_groups > n_groups || group_top < 1 ||
        (long long)keep_groups * (E / n_groups) < top || ((correction || n_groups > 1) && softmax_scores))
        return TNX_ERR_BAD_ARG;
    if (n_groups > 1 && E / n_groups > 64 && group_top > 1) return TNX_ERR_UNSUPPORTED;
    const RouterOptions ro{correction, n_groups, keep_groups, group_top, renorm_eps, weight_scale};
    const size_t smem = (size_t)(((W + 3) & ~3) + 3 * E) * sizeof(float);
    if (smem > 160 * 1024) return TNX_ERR_UNSUPPORTED;
#define GO(T, TW)                                                                                                       \
    do {                                                                                                                \
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_router_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tnx_launch_in_order(moe_router_kernel<T, TW>, dim3(N), dim3(128), smem, stream, (const T*)h, ld,         \
                                   (const TW*)router, token_request, ids, weights, W, E, top, softmax_scores, renormalize, ro); \
    } while (0)
    if (h_h16 && w_h16) GO(h16, h16);
    if (h_h16) GO(h16, float);
    if (w_h16) GO(float, h16);
    GO(float, float);
#undef GO
}

TNX_EXPORT int tnx_moe_experts(const void* h, int ld, const void* gate_up, const void* down, const int* ids,
                               const float* weights, void* y, float* per_pair, float* out, int N, int W, int F, int top,
                               int n_experts, float gate_max, float up_min, float up_max, float alpha, float up_shift,
                               int weight_on_input, int accumulate, int h_h16, int w_h16, int form, cudaStream_t stream) {
    // form 0: gate_up is [E, 2F, W] (gated experts); form 1: [E, F, W] (the up rows alone, y = relu(u)^2)
    if (N <= 0) return 0;
    if (W <= 0 || F <= 0 || top <= 0 || top > MAX_TOP || n_experts <= 0 || form < 0 || form > 1) return TNX_ERR_UNSUPPORTED;
    const int pairs = N * top;
    const size_t el = h_h16 ? 2 : 4;
    const size_t smem1 = (((size_t)MT * W * el + 15) & ~(size_t)15) + (size_t)pairs * sizeof(int);
    const size_t smem2 = (((size_t)MT * F * el + 15) & ~(size_t)15) + (size_t)pairs * sizeof(int);
    if (smem1 > 200 * 1024 || smem2 > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    ExpertMath m{gate_max, up_min, up_max, alpha, up_shift, weight_on_input, form};
    // slices that give every SM a few blocks of the experts that are chosen
    const int busy = n_experts < pairs ? n_experts : pairs;
    int per1 = 4; while (per1 < F && (long long)busy * ((F + per1 - 1) / per1) > 1024) per1 *= 2;
    int per2 = 4; while (per2 < W && (long long)busy * ((W + per2 - 1) / per2) > 1024) per2 *= 2;
    const dim3 g1(n_experts, (F + per1 - 1) / per1), g2(n_experts, (W + per2 - 1) / per2);
#define GO(T, TW)                                                                                                       \
    do {                                                                                                                \
        if (smem1 > 48 * 1024) cudaFuncSetAttribute(moe_gate_up_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1); \
        if (smem2 > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);    \
        int rc = tnx_launch_in_order(moe_gate_up_kernel<T, TW>, g1, dim3(128), smem1, stream, (const T*)h, ld,          \
                                     (const TW*)gate_up, ids, weights, (T*)y, W, F, top, pairs, per1, m);               \
        if (rc != 0) return rc;                                                                                         \
        rc = tnx_launch_in_order(moe_down_kernel<T, TW>, g2, dim3(128), smem2, stream, (const T*)y, (const TW*)down,    \
                                 ids, per_pair, W, F, pairs, per2);                                                     \
        if (rc != 0) return rc;                                                                                         \
        return tnx_launch_in_order(moe_sum_kernel, dim3(N, N >= 256 ? 1 : (W + 511) / 512), dim3(128), 0, stream, (const float*)per_pair, ids, weights, \
                                   out, W, top, accumulate, weight_on_input);                                           \
    } while (0)
    if (h_h16 && w_h16) GO(h16, h16);
    if (h_h16) GO(h16, float);
    if (w_h16) GO(float, h16);
    GO(float, float);
#undef GO
}
