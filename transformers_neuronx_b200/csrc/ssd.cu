// A selective state-space recurrence with one decay per head and token.  Per head h (group g = h / (H / G)), with x_t of
// P numbers, B_t and C_t of N numbers and a state S of N x P (32-bit, kept per request):
//     dt = softplus(dt_raw + dt_bias_h);   S <- exp(-exp(A_log_h) dt) S + dt B_t x_t^T;   y_t = S^T C_t + D_h x_t
// which is the recurrence of retention.cu with a decay and a key scale that change from token to token and with keys and
// queries (B and C) shared by the heads of a group: the scan itself is tnx_retention_scan with those options.  This file
// holds what lies around it.
//
// tnx_ssd_prep, per token, from the input projection's output `proj` (columns from col0 on: z [H P] | x [H P] | B [G N] |
//   C [G N] | dt [H]):  x, B and C pass one short causal convolution per channel,
//     y_t[c] = act(bias[c] + sum_j w[j, c] u_(t - taps + 1 + j)[c])       (zeros before position 0; the past comes from
//                                             this step's rows or from the request's state [slots, taps - 1, channels])
//   and leave as 32-bit x [N, H P], B and C [N, G N]; dt [N, H] and decay = exp(-exp(A_log) dt) [N, H] in 32-bit.
//   A request with one row shifts its convolution state here; requests with several rows are brought up to date by the
//   convolution library's state kernel afterwards.
// tnx_ssd_gate_norm, per (token, part): (y + D x) * act(z), divided by the root mean square of its part (the inner
//   width in `parts` equal parts, eps inside the root), times a weight over the inner width, written in the activation type.
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(256)
ssd_prep_kernel(const T* __restrict__ proj, int ld, int col0, const float* __restrict__ conv_w,
                const float* __restrict__ conv_b, int taps, T* state, const int* __restrict__ token_request,
                const int* __restrict__ positions, const int* __restrict__ q_start, const int* __restrict__ q_len,
                const int* __restrict__ state_slots, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                int act, float* __restrict__ x_out, float* __restrict__ b_out, float* __restrict__ c_out,
                float* __restrict__ dt_out, float* __restrict__ decay_out, int H, int P, int G, int Ns) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    const int req = token_request[n];
    if (req < 0) return;                              // a padded row of a captured step
    const int pos = positions[n], idx = n - q_start[req], slot = state_slots[req];
    const bool alone = q_len[req] == 1;
    const int keep = taps - 1, inner = H * P, gn = G * Ns, C = inner + 2 * gn;
    const T* row = proj + (size_t)n * ld + col0 + inner;       // the convolved channels begin behind z
    T* st = (keep > 0 && slot >= 0) ? state + (size_t)slot * keep * C : nullptr;
    const int first = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    for (int c = first; c < C; c += stride) {
        float past[MAX_TAPS];                         // past[b]: the projected value b positions back
        past[0] = to_float(row[c]);
        for (int b = 1; b < taps; ++b) {
            float v = 0.f;
            if (pos - b >= 0) {
                if (idx - b >= 0) v = to_float(row[c - (ptrdiff_t)b * ld]);
                else if (st) v = to_float(st[(size_t)(keep + idx - b) * C + c]);
            }
            past[b] = v;
        }
        float s = conv_b ? conv_b[c] : 0.f;
        for (int j = 0; j < taps; ++j) s = fmaf(conv_w[(size_t)j * C + c], past[taps - 1 - j], s);
        if (alone && st)                              // oldest first: what was one back is now two back
            for (int q = 0; q < keep; ++q) st[(size_t)q * C + c] = from_float<T>(past[keep - 1 - q]);
        s = apply_activation(s, act);
        if (c < inner) x_out[(size_t)n * inner + c] = s;
        else if (c < inner + gn) b_out[(size_t)n * gn + c - inner] = s;
        else c_out[(size_t)n * gn + c - inner - gn] = s;
    }
    for (int h = first; h < H; h += stride) {
        const float dt = softplus_f(to_float(proj[(size_t)n * ld + col0 + 2 * inner + 2 * gn + h]) + dt_bias[h]);
        dt_out[(size_t)n * H + h] = dt;
        decay_out[(size_t)n * H + h] = expf(-expf(a_log[h]) * dt);
    }
}

// The same with eight channels a thread (16-byte loads of the projections and the state, the taps' loads independent of
// one another): sizes and addresses in multiples of eight channels, so that no piece straddles x, B and C.  The sums
// are formed in the order of the one-channel form (the bias, then the oldest tap first).
template <typename T>
__global__ void __launch_bounds__(256)
ssd_prep_vec_kernel(const T* __restrict__ proj, int ld, int col0, const float* __restrict__ conv_w,
                    const float* __restrict__ conv_b, int taps, T* state, const int* __restrict__ token_request,
                    const int* __restrict__ positions, const int* __restrict__ q_start, const int* __restrict__ q_len,
                    const int* __restrict__ state_slots, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                    int act, float* __restrict__ x_out, float* __restrict__ b_out, float* __restrict__ c_out,
                    float* __restrict__ dt_out, float* __restrict__ decay_out, int H, int P, int G, int Ns) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    const int req = token_request[n];
    if (req < 0) return;                              // a padded row of a captured step
    const int pos = positions[n], idx = n - q_start[req], slot = state_slots[req];
    const bool alone = q_len[req] == 1;
    const int keep = taps - 1, inner = H * P, gn = G * Ns, C = inner + 2 * gn;
    const T* row = proj + (size_t)n * ld + col0 + inner;
    T* st = (keep > 0 && slot >= 0) ? state + (size_t)slot * keep * C : nullptr;
    const int first = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    for (int c = 8 * first; c < C; c += 8 * stride) {
        float s[8];
        if (conv_b) {
            const float4 b0 = *(const float4*)(conv_b + c), b1 = *(const float4*)(conv_b + c + 4);
            s[0] = b0.x; s[1] = b0.y; s[2] = b0.z; s[3] = b0.w; s[4] = b1.x; s[5] = b1.y; s[6] = b1.z; s[7] = b1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i] = 0.f;
        }
        for (int b = keep; b >= 0; --b) {             // oldest first
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
        float* dst = c < inner ? x_out + (size_t)n * inner + c
                               : (c < inner + gn ? b_out + (size_t)n * gn + (c - inner) : c_out + (size_t)n * gn + (c - inner - gn));
        *(float4*)dst = make_float4(s[0], s[1], s[2], s[3]);
        *(float4*)(dst + 4) = make_float4(s[4], s[5], s[6], s[7]);
    }
    for (int h = first; h < H; h += stride) {
        const float dt = softplus_f(to_float(proj[(size_t)n * ld + col0 + 2 * inner + 2 * gn + h]) + dt_bias[h]);
        dt_out[(size_t)n * H + h] = dt;
        decay_out[(size_t)n * H + h] = expf(-expf(a_log[h]) * dt);
    }
}

__device__ __forceinline__ void store4(float* p, const float (&v)[4]) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(h16* p, const float (&v)[4]) {
    uint2 raw;
    *(h16x2*)&raw.x = floats_to_h16x2(v[0], v[1]);
    *(h16x2*)&raw.y = floats_to_h16x2(v[2], v[3]);
    *(uint2*)p = raw;
}
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) { const float4 a = *(const float4*)p; v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; }
__device__ __forceinline__ void load4(const h16* p, float (&v)[4]) {
    const uint2 raw = *(const uint2*)p;
    const float2 a = h16x2_to_float2(*(const h16x2*)&raw.x), b = h16x2_to_float2(*(const h16x2*)&raw.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// VEC: four neighbouring channels a thread and pass (they lie in one head and one part; 16-byte loads of the 32-bit
// inputs, 8-byte ones of a 16-bit gate).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
ssd_gate_norm_kernel(const float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ skip,
                     const T* __restrict__ z, int z_ld, const int* __restrict__ token_request, const float* __restrict__ w,
                     float eps, int act, T* __restrict__ out, int out_ld, int inner, int P, int parts) {
    extern __shared__ __align__(16) float part[];     // the part's gated values between the two passes
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, g = blockIdx.y;
    if (token_request[n] < 0) return;
    const int size = inner / parts, c0 = g * size;
    float ss = 0.f;
    if (VEC) {
        for (int i = 4 * threadIdx.x; i < size; i += 4 * blockDim.x) {
            const int c = c0 + i;
            float v[4], xv[4], zv[4];
            load4(y + (size_t)n * inner + c, v);
            if (skip) {
                load4(x + (size_t)n * inner + c, xv);
                const float d = skip[c / P];
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = fmaf(d, xv[e], v[e]);
            }
            load4(z + (size_t)n * z_ld + c, zv);
#pragma unroll
            for (int e = 0; e < 4; ++e) { v[e] *= apply_activation(zv[e], act); ss = fmaf(v[e], v[e], ss); }
            *(float4*)(part + i) = make_float4(v[0], v[1], v[2], v[3]);
        }
    } else {
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            const int c = c0 + i;
            float v = y[(size_t)n * inner + c];
            if (skip) v = fmaf(skip[c / P], x[(size_t)n * inner + c], v);
            v *= apply_activation(to_float(z[(size_t)n * z_ld + c]), act);
            part[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)size + eps);
    if (VEC) {
        for (int i = 4 * threadIdx.x; i < size; i += 4 * blockDim.x) {      // a thread reads back what it wrote itself
            const float4 v = *(const float4*)(part + i);
            float o[4] = {v.x * rinv, v.y * rinv, v.z * rinv, v.w * rinv};
            if (w) {
                const float4 g4 = *(const float4*)(w + c0 + i);
                o[0] *= g4.x; o[1] *= g4.y; o[2] *= g4.z; o[3] *= g4.w;
            }
            store4(out + (size_t)n * out_ld + c0 + i, o);
        }
    } else {
        for (int i = threadIdx.x; i < size; i += blockDim.x)
            out[(size_t)n * out_ld + c0 + i] = from_float<T>(part[i] * rinv * (w ? w[c0 + i] : 1.f));
    }
}
}  // namespace

TNX_EXPORT int tnx_ssd_prep(const void* proj, int ld, int col0, const float* conv_w, const float* conv_b, int taps,
                            void* state, const int* token_request, const int* positions, const int* q_start,
                            const int* q_len, const int* state_slots, const float* a_log, const float* dt_bias, int act,
                            float* x_out, float* b_out, float* c_out, float* dt_out, float* decay_out, int N, int H, int P,
                            int G, int Ns, int is_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || P <= 0 || G <= 0 || Ns <= 0 || H % G || taps < 1 || taps > MAX_TAPS || !conv_w || act < 0 ||
        act >= TNX_ACT_COUNT)
        return TNX_ERR_BAD_ARG;
    if (taps > 1 && !state) return TNX_ERR_BAD_ARG;
    const int C = H * P + 2 * G * Ns;
    // a prompt's tokens: one block a token; the few tokens of a decode step: a token's channels over several blocks
    int ny = 1;
    if (N < 256) { ny = (C + 255) / 256; if (ny > 16) ny = 16; }
    // eight channels a thread where every piece of eight is whole, inside one of x, B and C, and 16-byte aligned
    const size_t el = is_h16 ? 2 : 4;
    const bool vec = (H * P) % 8 == 0 && (G * Ns) % 8 == 0 && ld % 8 == 0 && (col0 + H * P) % 8 == 0 &&
                     ((uintptr_t)proj % 16) == 0 && ((uintptr_t)state % 16) == 0 && ((uintptr_t)conv_w % 16) == 0 &&
                     ((uintptr_t)conv_b % 16) == 0 && (((uintptr_t)x_out | (uintptr_t)b_out | (uintptr_t)c_out) % 16) == 0 &&
                     (ld * el) % 16 == 0;
    if (vec) {
        int vy = 1;
        if (N < 256) { vy = (C / 8 + 255) / 256; if (vy > 16) vy = 16; }
        const dim3 vgrid(N, vy);
        // few channels a token: smaller blocks, so that a block's threads all have a piece
        const int threads = C / 8 >= 256 * vy ? 256 : (C / 8 >= 128 * vy ? 128 : 64);
        if (is_h16)
            return tnx_launch_in_order(ssd_prep_vec_kernel<h16>, vgrid, dim3(threads), 0, stream, (const h16*)proj, ld, col0,
                                       conv_w, conv_b, taps, (h16*)state, token_request, positions, q_start, q_len,
                                       state_slots, a_log, dt_bias, act, x_out, b_out, c_out, dt_out, decay_out, H, P, G, Ns);
        return tnx_launch_in_order(ssd_prep_vec_kernel<float>, vgrid, dim3(threads), 0, stream, (const float*)proj, ld, col0,
                                   conv_w, conv_b, taps, (float*)state, token_request, positions, q_start, q_len,
                                   state_slots, a_log, dt_bias, act, x_out, b_out, c_out, dt_out, decay_out, H, P, G, Ns);
    }
    const dim3 grid(N, ny);
    if (is_h16)
        return tnx_launch_in_order(ssd_prep_kernel<h16>, grid, dim3(256), 0, stream, (const h16*)proj, ld, col0, conv_w,
                                   conv_b, taps, (h16*)state, token_request, positions, q_start, q_len, state_slots, a_log,
                                   dt_bias, act, x_out, b_out, c_out, dt_out, decay_out, H, P, G, Ns);
    return tnx_launch_in_order(ssd_prep_kernel<float>, grid, dim3(256), 0, stream, (const float*)proj, ld, col0, conv_w,
                               conv_b, taps, (float*)state, token_request, positions, q_start, q_len, state_slots, a_log,
                               dt_bias, act, x_out, b_out, c_out, dt_out, decay_out, H, P, G, Ns);
}

TNX_EXPORT int tnx_ssd_gate_norm(const float* y, const float* x, const float* skip, const void* z, int z_ld,
                                 const int* token_request, const float* w, float eps, int act, void* out, int out_ld, int N,
                                 int inner, int P, int parts, int is_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (inner <= 0 || P <= 0 || parts <= 0 || inner % parts || out_ld < inner || act < 0 || act >= TNX_ACT_COUNT || (skip && !x))
        return TNX_ERR_BAD_ARG;
    const int size = inner / parts;
    const size_t smem = (size_t)size * sizeof(float);
    if (smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const size_t el = is_h16 ? 2 : 4;
    const bool vec = size % 4 == 0 && P % 4 == 0 && z_ld % 4 == 0 && out_ld % 4 == 0 &&
                     !(((uintptr_t)y | (uintptr_t)x | (uintptr_t)w) & 15) && !(((uintptr_t)z | (uintptr_t)out) & (4 * el - 1));
    const int per = vec ? 4 : 1;
    const int threads = size >= 1024 * per ? 256 : (size >= 256 * per ? 128 : 64);
    const dim3 grid(N, parts);
#define GO(T)                                                                                                           \
    do {                                                                                                                \
        if (smem > 48 * 1024) {                                                                                         \
            cudaFuncSetAttribute(ssd_gate_norm_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            cudaFuncSetAttribute(ssd_gate_norm_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        }                                                                                                               \
        if (vec)                                                                                                        \
            return tnx_launch_in_order(ssd_gate_norm_kernel<T, true>, grid, dim3(threads), smem, stream, y, x, skip,    \
                                       (const T*)z, z_ld, token_request, w, eps, act, (T*)out, out_ld, inner, P, parts); \
        return tnx_launch_in_order(ssd_gate_norm_kernel<T, false>, grid, dim3(threads), smem, stream, y, x, skip,       \
                                   (const T*)z, z_ld, token_request, w, eps, act, (T*)out, out_ld, inner, P, parts);    \
    } while (0)
    if (is_h16) GO(h16);
    GO(float);
#undef GO
}
