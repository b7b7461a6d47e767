// A recurrence with an error-correcting write ("delta rule") and a decay per head and key channel.  Per head, with
// q_t, k_t of k_dim numbers, v_t of v_dim numbers and a state S of k_dim x v_dim (32-bit, kept per request):
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// so the read-out sees the current token's write.  Query/key heads may be shared by groups of heads (G of them for H
// heads: head h uses q/k head h / (H / G)).
//
// tnx_delta_prep, per token (one thread block for a prompt's tokens; several for the few tokens of a decode step, which
//   share the token's heads and channels, so that eight tokens still fill the device): from the projections' output
//   (queries, keys and values side by side from column col0 on: G*dk, G*dk, H*dv channels)
//     y_t[c] = act(sum_j w[j, c] u_(t - taps + 1 + j)[c])        the short causal convolution (zeros before position 0;
//                                                                 the past comes from this step's rows or from the
//                                                                 request's state [slots, taps - 1, channels])
//     q, k per head: y / sqrt(sum(y^2) + unit_eps), q times q_scale;  v = y
//     beta[h] = sigmoid(proj[b_off + h]);   g[h, i] = exp(-exp(a_log[h]) * softplus(a[h * dk + i] + dt_bias[h * dk + i]))
//   Everything after the loads is 32-bit and stays 32-bit: q, k, v, beta and g are written as floats.  A request with
//   one row shifts its convolution state here; requests with several rows are brought up to date by the convolution
//   library's state kernel afterwards.
// tnx_delta_scan: a thread block owns C columns (value dims) of one head of one request and walks the request's tokens
//   of this step in order, the state's columns in registers: a column's k_dim rows are spread over R adjacent lanes,
//   which add their partial sums of S^T k, S^T q and q.k with shuffles (one round for all three: o = (gS)^T q + (q.k) u).
//   The tokens' inputs reach shared memory by asynchronous copies, a stage ahead of the walk.
//   The state is stored [slot, head, v_dim, k_dim] (a column's rows side by side).
#include "common.cuh"

namespace {

constexpr int PREP_MAX_TAPS = 8;
constexpr int PREP_FILL_BLOCKS = 2 * 148;   // blocks that fill the device: two an SM

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(256)
delta_prep_kernel(const T* __restrict__ proj, int ld, int col0, int b_off, const float* __restrict__ a, int a_ld,
                  const float* __restrict__ conv_w, int taps, T* state, const int* __restrict__ token_request,
                  const int* __restrict__ positions, const int* __restrict__ q_start, const int* __restrict__ q_len,
                  const int* __restrict__ state_slots, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  float unit_eps, float q_scale, int act, float* __restrict__ q_out, float* __restrict__ k_out,
                  float* __restrict__ v_out, float* __restrict__ beta_out, float* __restrict__ g_out, int H, int G, int dk,
                  int dv) {
    extern __shared__ float y[];                      // a query or key head's convolved channels, per warp
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    const int req = token_request[n];
    if (req < 0) return;                              // a padded row of a captured step
    const int pos = positions[n], idx = n - q_start[req], slot = state_slots[req];
    const bool alone = q_len[req] == 1;
    const int keep = taps - 1, nqk = 2 * G * dk, C = nqk + H * dv;
    const T* row = proj + (size_t)n * ld + col0;
    T* st = (keep > 0 && slot >= 0) ? state + (size_t)slot * keep * C : nullptr;
    auto conv = [&](int c) -> float {                 // channel c of this token: convolution, state shift, activation
        float past[PREP_MAX_TAPS];                    // past[b]: the projected value b positions back
        past[0] = to_float(row[c]);
        for (int b = 1; b < taps; ++b) {
            float v = 0.f;
            if (pos - b >= 0) {
                if (idx - b >= 0) v = to_float(row[c - (ptrdiff_t)b * ld]);
                else if (st) v = to_float(st[(size_t)(keep + idx - b) * C + c]);
            }
            past[b] = v;
        }
        float s = 0.f;
        for (int j = 0; j < taps; ++j) s = fmaf(conv_w[(size_t)j * C + c], past[taps - 1 - j], s);
        if (alone && st)                              // oldest first: what was one back is now two back
            for (int q = 0; q < keep; ++q) st[(size_t)q * C + c] = from_float<T>(past[keep - 1 - q]);
        return apply_activation(s, act);
    };
    // The token's work is spread over gridDim.y blocks: heads of q and k a warp each (unit vectors), the rest a thread
    // per channel.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* mine = y + warp * dk;
    for (int u = blockIdx.y * warps + warp; u < 2 * G; u += gridDim.y * warps) {      // the heads of q, then those of k
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) {
            const float x = conv(u * dk + i);
            mine[i] = x;
            ss = fmaf(x, x, ss);
        }
        const float rinv = (u < G ? q_scale : 1.f) / sqrtf(warp_sum(ss) + unit_eps);
        float* dst = (u < G ? q_out + (size_t)n * G * dk + u * dk : k_out + (size_t)n * G * dk + (u - G) * dk);
        for (int i = lane; i < dk; i += 32) dst[i] = mine[i] * rinv;      // a lane reads back what it wrote itself
    }
    const int first = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    for (int c = first; c < H * dv; c += stride) v_out[(size_t)n * H * dv + c] = conv(nqk + c);
    for (int h = first; h < H; h += stride)
        beta_out[(size_t)n * H + h] = 1.f / (1.f + expf(-to_float(proj[(size_t)n * ld + b_off + h])));
    for (int c = first; c < H * dk; c += stride) {
        const float rate = expf(a_log[c / dk]);
        g_out[(size_t)n * H * dk + c] = expf(-rate * softplus_f(a[(size_t)n * a_ld + c] + dt_bias[c]));
    }
}

// The same with eight channels a thread (16-byte loads of the projections and the state, the taps' loads independent of
// one another): sizes and addresses in multiples of eight channels.
template <typename T>
__global__ void __launch_bounds__(256)
delta_prep_vec_kernel(const T* __restrict__ proj, int ld, int col0, int b_off, const float* __restrict__ a, int a_ld,
                  const float* __restrict__ conv_w, int taps, T* state, const int* __restrict__ token_request,
                  const int* __restrict__ positions, const int* __restrict__ q_start, const int* __restrict__ q_len,
                  const int* __restrict__ state_slots, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  float unit_eps, float q_scale, int act, float* __restrict__ q_out, float* __restrict__ k_out,
                  float* __restrict__ v_out, float* __restrict__ beta_out, float* __restrict__ g_out, int H, int G, int dk,
                  int dv) {
    extern __shared__ float y[];                      // a query or key head's convolved channels, per warp
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    const int req = token_request[n];
    if (req < 0) return;                              // a padded row of a captured step
    const int pos = positions[n], idx = n - q_start[req], slot = state_slots[req];
    const bool alone = q_len[req] == 1;
    const int keep = taps - 1, nqk = 2 * G * dk, C = nqk + H * dv;
    const T* row = proj + (size_t)n * ld + col0;
    T* st = (keep > 0 && slot >= 0) ? state + (size_t)slot * keep * C : nullptr;
    auto conv8 = [&](int c, float (&s)[8]) {          // channels c .. c + 7: convolution, state shift, activation
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = 0.f;
        for (int b = keep; b >= 0; --b) {             // oldest first, as the one-channel form adds them
            const T* src = row + c;                   // the value b positions back: this step's rows, the state, or zero
            if (b > 0) {
                if (pos - b < 0) src = nullptr;
                else if (idx - b >= 0) src = row + c - (ptrdiff_t)b * ld;
                else src = st ? st + (size_t)(keep + idx - b) * C + c : nullptr;
            }
            Vec8<T> x;
            if (src) x.load(src); else x.zero();
            const float* w = conv_w + (size_t)(keep - b) * C + c;
            const float4 w0 = *(const float4*)w, w1 = *(const float4*)(w + 4);
            float xv[8];
            x.get(xv);
            s[0] = fmaf(w0.x, xv[0], s[0]); s[1] = fmaf(w0.y, xv[1], s[1]); s[2] = fmaf(w0.z, xv[2], s[2]);
            s[3] = fmaf(w0.w, xv[3], s[3]); s[4] = fmaf(w1.x, xv[4], s[4]); s[5] = fmaf(w1.y, xv[5], s[5]);
            s[6] = fmaf(w1.z, xv[6], s[6]); s[7] = fmaf(w1.w, xv[7], s[7]);
            // a request's single row moves its past on: what is b back now is b + 1 back for the next token (the slot
            // written here was read one round ago)
            if (alone && st && b < keep) x.store(st + (size_t)(keep - 1 - b) * C + c);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = apply_activation(s[i], act);
    };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* mine = y + warp * dk;
    for (int u = blockIdx.y * warps + warp; u < 2 * G; u += gridDim.y * warps) {      // the heads of q, then those of k
        float ss = 0.f;
        for (int i = 8 * lane; i < dk; i += 256) {
            float s[8];
            conv8(u * dk + i, s);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(s[e], s[e], ss);
            *(float4*)(mine + i) = make_float4(s[0], s[1], s[2], s[3]);
            *(float4*)(mine + i + 4) = make_float4(s[4], s[5], s[6], s[7]);
        }
        const float rinv = (u < G ? q_scale : 1.f) / sqrtf(warp_sum(ss) + unit_eps);
        float* dst = (u < G ? q_out + (size_t)n * G * dk + u * dk : k_out + (size_t)n * G * dk + (u - G) * dk);
        for (int i = 8 * lane; i < dk; i += 256) {    // a lane reads back what it wrote itself
            float4 a0 = *(const float4*)(mine + i), a1 = *(const float4*)(mine + i + 4);
            a0.x *= rinv; a0.y *= rinv; a0.z *= rinv; a0.w *= rinv; a1.x *= rinv; a1.y *= rinv; a1.z *= rinv; a1.w *= rinv;
            *(float4*)(dst + i) = a0;
            *(float4*)(dst + i + 4) = a1;
        }
    }
    const int first = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    for (int c = 8 * first; c < H * dv; c += 8 * stride) {
        float s[8];
        conv8(nqk + c, s);
        float* dst = v_out + (size_t)n * H * dv + c;
        *(float4*)dst = make_float4(s[0], s[1], s[2], s[3]);
        *(float4*)(dst + 4) = make_float4(s[4], s[5], s[6], s[7]);
    }
    for (int h = first; h < H; h += stride)
        beta_out[(size_t)n * H + h] = 1.f / (1.f + expf(-to_float(proj[(size_t)n * ld + b_off + h])));
    for (int c = 4 * first; c < H * dk; c += 4 * stride) {          // four channels of one head (dk is a multiple of 8)
        const float rate = expf(a_log[c / dk]);
        const float4 x = *(const float4*)(a + (size_t)n * a_ld + c), bias = *(const float4*)(dt_bias + c);
        *(float4*)(g_out + (size_t)n * H * dk + c) =
            make_float4(expf(-rate * softplus_f(x.x + bias.x)), expf(-rate * softplus_f(x.y + bias.y)),
                        expf(-rate * softplus_f(x.z + bias.z)), expf(-rate * softplus_f(x.w + bias.w)));
    }
}

// tokens whose inputs are staged in shared memory at a time, in each of two buffers (24 KB of keys, queries and decays)
__host__ __device__ constexpr int scan_stage(int dkp) { return dkp > 128 ? 4 : dkp > 64 ? 8 : 16; }

// Asynchronous copies global -> shared; `bytes_src` 0 fills the destination with zeros and reads nothing.
__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool take) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(take ? 4u : 0u) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool take) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(take ? 16u : 0u) : "memory");
}

// KPT: rows of a column one thread keeps; R: lanes a column's rows are spread over (KPT * R >= k_dim); a block of 128
// threads owns 128 / R columns.  The tokens' inputs come in stages through two buffers: while one stage is walked, the
// next one's copies are in flight, so the walk waits for memory once, at the first stage.  VEC: k_dim is a multiple
// of 4 and the rows are 16-byte aligned (16-byte copies).
template <int KPT, int R, bool VEC>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ beta, const float* __restrict__ g, float* __restrict__ state,
                  const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ state_slots,
                  float* __restrict__ out, int H, int G, int dk, int dv) {
    constexpr int DKP = KPT * R, C = 128 / R, ST = scan_stage(KPT * R);
    __shared__ __align__(16) float qs[2][ST][DKP], ks[2][ST][DKP], gs[2][ST][DKP];
    __shared__ float vs[2][ST][C], bs[2][ST];
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.z, h = blockIdx.y;
    const int len = q_len[req];
    if (len <= 0) return;                             // a padded request of a captured batch
    const int slot = state_slots[req];
    if (slot < 0) return;
    const int t_first = q_start[req], kvh = h / (H / G);
    const int jl = threadIdx.x / R, r = threadIdx.x % R;
    const int j = blockIdx.x * C + jl;
    const bool col = j < dv;

    auto fetch = [&](int t0, int buf) {               // the inputs of tokens t0 .. t0 + ST - 1 of this request's rows
        const int nt = min(ST, len - t0);
        if (VEC) {
            for (int e = threadIdx.x; e < nt * (DKP / 4); e += 128) {
                const int tt = e / (DKP / 4), i = (e % (DKP / 4)) * 4;
                const size_t t = (size_t)(t_first + t0 + tt);
                const bool in = i < dk;
                cp_async16(&qs[buf][tt][i], in ? q + (t * G + kvh) * dk + i : q, in);
                cp_async16(&ks[buf][tt][i], in ? k + (t * G + kvh) * dk + i : k, in);
                cp_async16(&gs[buf][tt][i], in ? g + (t * H + h) * dk + i : g, in);
            }
        } else {
            for (int e = threadIdx.x; e < nt * DKP; e += 128) {
                const int tt = e / DKP, i = e % DKP;
                const size_t t = (size_t)(t_first + t0 + tt);
                const bool in = i < dk;
                cp_async4(&qs[buf][tt][i], in ? q + (t * G + kvh) * dk + i : q, in);
                cp_async4(&ks[buf][tt][i], in ? k + (t * G + kvh) * dk + i : k, in);
                cp_async4(&gs[buf][tt][i], in ? g + (t * H + h) * dk + i : g, in);
            }
        }
        for (int e = threadIdx.x; e < nt * C; e += 128) {
            const int tt = e / C, c = blockIdx.x * C + e % C;
            cp_async4(&vs[buf][tt][e % C], c < dv ? v + ((size_t)(t_first + t0 + tt) * H + h) * dv + c : v, c < dv);
        }
        if (threadIdx.x < nt) cp_async4(&bs[buf][threadIdx.x], beta + (size_t)(t_first + t0 + threadIdx.x) * H + h, true);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    fetch(0, 0);
    float* st = state + (((size_t)slot * H + h) * dv + (col ? j : 0)) * dk;
    float S[KPT];
#pragma unroll
    for (int m = 0; m < KPT; ++m) S[m] = (col && r + R * m < dk) ? st[r + R * m] : 0.f;
    int buf = 0;
    for (int t0 = 0; t0 < len; t0 += ST, buf ^= 1) {
        const int nt = min(ST, len - t0);
        if (t0 + ST < len) {
            fetch(t0 + ST, buf ^ 1);                  // the buffer that the stage before this one used: all have left it
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                              // every thread's copies of this stage have landed
        for (int tt = 0; tt < nt; ++tt) {
            float sk0 = 0.f, sk1 = 0.f, sq0 = 0.f, sq1 = 0.f, qk = 0.f;
            float Sg[KPT];
            // the decayed state first, then its products with k and q, in two chains each (half the dependent adds)
#pragma unroll
            for (int m = 0; m < KPT; ++m) {
                const int i = r + R * m;
                const float kk = ks[buf][tt][i], qq = qs[buf][tt][i], gg = gs[buf][tt][i];
                Sg[m] = S[m] * gg;
                if (m & 1) { sk1 = fmaf(kk, Sg[m], sk1); sq1 = fmaf(qq, Sg[m], sq1); }
                else { sk0 = fmaf(kk, Sg[m], sk0); sq0 = fmaf(qq, Sg[m], sq0); }
                qk = fmaf(qq, kk, qk);
            }
            float sk = sk0 + sk1, sq = sq0 + sq1;
#pragma unroll
            for (int o = R >> 1; o > 0; o >>= 1) {    // the R lanes of a column are neighbours in one warp
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                qk += __shfl_xor_sync(0xffffffffu, qk, o);
            }
            const float u = bs[buf][tt] * (vs[buf][tt][jl] - sk);
#pragma unroll
            for (int m = 0; m < KPT; ++m) S[m] = fmaf(ks[buf][tt][r + R * m], u, Sg[m]);
            if (r == 0 && col) out[((size_t)(t_first + t0 + tt) * H + h) * dv + j] = fmaf(qk, u, sq);
        }
        __syncthreads();                              // the stage is no longer read: the next fetch may overwrite it
    }
    if (col) {
#pragma unroll
        for (int m = 0; m < KPT; ++m)
            if (r + R * m < dk) st[r + R * m] = S[m];
    }
}

}  // namespace

TNX_EXPORT int tnx_delta_prep(const void* proj, int ld, int col0, int b_off, const float* a, int a_ld, const float* conv_w,
                              int taps, void* state, const int* token_request, const int* positions, const int* q_start,
                              const int* q_len, const int* state_slots, const float* a_log, const float* dt_bias,
                              float unit_eps, float q_scale, int act, float* q_out, float* k_out, float* v_out,
                              float* beta_out, float* g_out, int n_tokens, int H, int G, int dk, int dv, int is_h16,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1 || taps > PREP_MAX_TAPS || !conv_w ||
        (taps > 1 && !state) || act < 0 || act >= TNX_ACT_COUNT)
        return TNX_ERR_BAD_ARG;
    const size_t smem = (size_t)8 * dk * sizeof(float);
    if (smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    // few tokens: a token's channels over several blocks, so that a step of single tokens fills the device
    const int most = max(1, max((2 * G + 7) / 8, (H * max(dk, dv) + 255) / 256));
    const int parts = min(most, max(1, (PREP_FILL_BLOCKS + n_tokens - 1) / n_tokens));
    const bool vec = dk % 8 == 0 && dv % 8 == 0 && ld % 8 == 0 && col0 % 8 == 0 && a_ld % 4 == 0 &&
                     !(((uintptr_t)proj | (uintptr_t)state | (uintptr_t)conv_w | (uintptr_t)a | (uintptr_t)dt_bias |
                        (uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)v_out | (uintptr_t)g_out) & 15);
#define DPREP(T)                                                                                                        \
    do {                                                                                                                \
        auto kernel = vec ? delta_prep_vec_kernel<T> : delta_prep_kernel<T>;                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        return tnx_launch_in_order(kernel, dim3(n_tokens, parts), dim3(256), smem, stream, (const T*)proj, ld, col0,    \
                                   b_off, a, a_ld, conv_w, taps, (T*)state, token_request, positions, q_start, q_len,   \
                                   state_slots, a_log, dt_bias, unit_eps, q_scale, act, q_out, k_out, v_out, beta_out,  \
                                   g_out, H, G, dk, dv);                                                                \
    } while (0)
    if (is_h16) DPREP(h16);
    DPREP(float);
#undef DPREP
}

TNX_EXPORT int tnx_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* g,
                              float* state, const int* q_start, const int* q_len, const int* state_slots, float* out,
                              int n_requests, int H, int G, int dk, int dv, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0) return TNX_ERR_BAD_ARG;
#define DSCAN(KPT, R)                                                                                                   \
    do {                                                                                                                \
        const int C = 128 / (R);                                                                                        \
        const dim3 grid((dv + C - 1) / C, H, n_requests);                                                               \
        if (vec)                                                                                                        \
            return tnx_launch_in_order(delta_scan_kernel<KPT, R, true>, grid, dim3(128), 0, stream, q, k, v, beta, g,   \
                                       state, q_start, q_len, state_slots, out, H, G, dk, dv);                          \
        return tnx_launch_in_order(delta_scan_kernel<KPT, R, false>, grid, dim3(128), 0, stream, q, k, v, beta, g,      \
                                   state, q_start, q_len, state_slots, out, H, G, dk, dv);                              \
    } while (0)
    const bool vec = dk % 4 == 0 && !(((uintptr_t)q | (uintptr_t)k | (uintptr_t)g) & 15);
    if (dk <= 16) DSCAN(4, 4);
    if (dk <= 32) DSCAN(4, 8);
    if (dk <= 64) DSCAN(8, 8);
    if (dk <= 128) DSCAN(8, 16);
    if (dk <= 256) DSCAN(16, 16);
    return TNX_ERR_UNSUPPORTED;
#undef DSCAN
}
