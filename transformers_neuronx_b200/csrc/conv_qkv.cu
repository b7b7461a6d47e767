// What lies between an attention mixer's projections and its attention kernel when the projections pass through
// a short causal convolution over time:
//
//   u_t[c]   the projection's output (bias included) of channel c at position t of the request; zero before position 0
//   y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]                     j = 0 .. taps - 1   (no convolution: y = u)
//   queries and keys, per head of `dk` channels:  y / sqrt(mean(y^2) + eps) * g[c]   (g: one weight vector for all heads)
//   then the first rot_dims channels of each head turned by the position: pairs (2i, 2i + 1) (interleaved) or
//   (i, i + rot_dims / 2) (halves), (a, b) -> (a cos - b sin, b cos + a sin) * magnitude, angle = t * inv_freq[i]
//   values: y only.
//
// Everything after the loads is 32-bit (the angle is position x frequency in 32-bit, sincosf); the results are
// written in the activation type with `D` channels a head, the rest zero, as the attention kernels and the pages want
// them.  The last taps - 1 projected values of every channel are the request's state ([slots, taps - 1, channels], in
// the projection's type, oldest first): a token whose predecessors are not among this step's rows reads them from
// there, so the result does not depend on how the request was cut into steps.  A request with one row updates its
// state in the same kernel (no other row reads it); requests with several rows are brought up to date by
// conv_state_update_kernel, launched after every row has read the old state.
//
// Two kernels do this.  conv_norm_rotate_vec_kernel takes head sizes that are multiples of 8 with interleaved pairs (or no
// rotation) and up to four taps: a lane owns 8 consecutive channels of a head (16-byte loads and stores in a 16-bit type,
// four pairs of a rotation inside the lane), the dims/8 lanes of a head sit side by side in a warp, several heads a warp.
// conv_norm_rotate_kernel takes everything else: one thread block per token, one warp per head at a time, a lane owns
// the pairs (2 lane, 2 lane + 1) + 64 r of the head.
#include "common.cuh"

namespace {
constexpr int MAX_R = 4;            // a head has at most 64 * MAX_R channels
constexpr int MAX_TAPS = 8;

template <typename T>
struct ConvPrep {
    const T* proj; int ld; int col0;             // the mixer's projections begin at column col0: queries, keys, values
    const float* conv_w; int taps;              // [taps, channels] or null (no convolution; taps is 1 then)
    T* state;                                   // [slots, taps - 1, channels]
    const int* token_request; const int* positions; const int* q_start; const int* q_len; const int* state_slots;
    const float* q_norm; const float* k_norm; float eps;      // [dk] each, or null
    const float* inv_freq; int rot_dims; int interleaved; float magnitude;
    T* q_out; T* k_out; T* v_out;
    int H, G, dk, dv, D;                        // G = 0: the mixer has no keys and values of its own
    int channels;
};

template <typename T>
__global__ void __launch_bounds__(128) conv_norm_rotate_kernel(const ConvPrep<T> p) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int req = p.token_request[n];
    if (req < 0) return;                                    // a padded row of a captured step
    const int pos = p.positions[n], idx = n - p.q_start[req], slot = p.state_slots[req];
    const bool alone = p.q_len[req] == 1;
    const int taps = p.taps, keep = taps - 1;
    const T* row = p.proj + (size_t)n * p.ld + p.col0;
    T* st = (keep > 0 && slot >= 0) ? p.state + (size_t)slot * keep * p.channels : nullptr;
    const int units = p.H + 2 * p.G;
    for (int u = warp; u < units; u += 4) {
        const int kind = u < p.H ? 0 : (u < p.H + p.G ? 1 : 2);
        const int head = kind == 0 ? u : (kind == 1 ? u - p.H : u - p.H - p.G);
        const int dims = kind == 2 ? p.dv : p.dk;
        const int base = kind == 0 ? head * p.dk : (kind == 1 ? p.H * p.dk + head * p.dk : (p.H + p.G) * p.dk + head * p.dv);
        float val[MAX_R][2];
        float ssq = 0.f;
#pragma unroll
        for (int r = 0; r < MAX_R; ++r)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 2 * lane + 64 * r + e;
                float y = 0.f;
                if (c < dims) {
                    const int ch = base + c;
                    const float cur = to_float(row[ch]);
                    if (p.conv_w == nullptr) {
                        y = cur;
                    } else {
                        float past[MAX_TAPS];                   // past[b]: the projected value b positions back
                        past[0] = cur;
                        for (int b = 1; b < taps; ++b) {
                            float v = 0.f;
                            if (pos - b >= 0) {
                                if (idx - b >= 0) v = to_float(row[ch - (ptrdiff_t)b * p.ld]);
                                else if (st) v = to_float(st[(size_t)(keep + idx - b) * p.channels + ch]);
                            }
                            past[b] = v;
                        }
                        for (int j = 0; j < taps; ++j) y = fmaf(p.conv_w[(size_t)j * p.channels + ch], past[taps - 1 - j], y);
                        if (alone && st) {                      // oldest first: what was one back is now two back
                            for (int s = 0; s < keep; ++s)
                                st[(size_t)s * p.channels + ch] = from_float<T>(past[keep - 1 - s]);
                        }
                    }
                }
                val[r][e] = y;
                ssq = fmaf(y, y, ssq);
            }
        T* out = (kind == 0 ? p.q_out + (size_t)n * p.H * p.D : (kind == 1 ? p.k_out : p.v_out) + (size_t)n * p.G * p.D) +
                 (size_t)head * p.D;
        const float* g = kind == 0 ? p.q_norm : (kind == 1 ? p.k_norm : nullptr);
        if (kind != 2) {
            if (g != nullptr) {
                const float rinv = 1.0f / sqrtf(warp_sum(ssq) / (float)dims + p.eps);
#pragma unroll
                for (int r = 0; r < MAX_R; ++r)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int c = 2 * lane + 64 * r + e;
                        if (c < dims) val[r][e] *= rinv * g[c];
                    }
            }
            if (p.rot_dims > 0 && p.interleaved) {
#pragma unroll
                for (int r = 0; r < MAX_R; ++r) {
                    const int c = 2 * lane + 64 * r;
                    if (c + 1 < p.rot_dims) {
                        float sn, cs;
                        sincosf((float)pos * p.inv_freq[c >> 1], &sn, &cs);
                        sn *= p.magnitude; cs *= p.magnitude;
                        const float a = val[r][0], b = val[r][1];
                        val[r][0] = a * cs - b * sn;
                        val[r][1] = b * cs + a * sn;
                    }
                }
            }
        }
        if (kind != 2 && p.rot_dims > 0 && !p.interleaved) {
            // halves: channel i turns with channel i + rot_dims / 2, which another lane may own: through shared memory
            __shared__ float sh[4][64 * MAX_R];
            float* mine = sh[warp];
#pragma unroll
            for (int r = 0; r < MAX_R; ++r)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = 2 * lane + 64 * r + e;
                    if (c < dims) mine[c] = val[r][e];
                }
            __syncwarp();
            const int half = p.rot_dims / 2;
#pragma unroll
            for (int r = 0; r < MAX_R; ++r)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = 2 * lane + 64 * r + e;
                    if (c < p.rot_dims && c < dims) {
                        const int i = c < half ? c : c - half;
                        float sn, cs;
                        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
                        sn *= p.magnitude; cs *= p.magnitude;
                        const float a = mine[i], b = mine[i + half];
                        val[r][e] = c < half ? a * cs - b * sn : b * cs + a * sn;
                    }
                }
            __syncwarp();
        }
#pragma unroll
        for (int r = 0; r < MAX_R; ++r)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 2 * lane + 64 * r + e;
                if (c < p.D) out[c] = from_float<T>(c < dims ? val[r][e] : 0.f);
            }
    }
}

// TAPS: the convolution's taps, 1 when there is none.  grid (tokens, groups of four warps); a warp takes 32 / (dims / 8)
// heads: first those of queries and keys (which lie side by side in the projection and have one size), then the values'.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128) conv_norm_rotate_vec_kernel(const ConvPrep<T> p) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, lane = threadIdx.x & 31;
    const int req = p.token_request[n];
    if (req < 0) return;                                    // a padded row of a captured step
    const int pos = p.positions[n];
    // the token's sines and cosines once for all heads of the block (they were a third of the kernel's instructions when
    // every lane computed its own four)
    __shared__ float2 turn[32 * MAX_R];
    for (int i = threadIdx.x; 2 * i < p.rot_dims; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
        turn[i] = make_float2(cs * p.magnitude, sn * p.magnitude);
    }
    __syncthreads();
    const int Lk = p.dk >> 3, Lv = p.dv >> 3;
    const int per_k = 32 / Lk, per_v = Lv ? 32 / Lv : 1, n_qk = p.H + p.G;
    const int warps_qk = (n_qk + per_k - 1) / per_k, warps_v = p.G ? (p.G + per_v - 1) / per_v : 0;
    const int w = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (w >= warps_qk + warps_v) return;
    const bool values = w >= warps_qk;
    const int L = values ? Lv : Lk, dims = values ? p.dv : p.dk;
    const int unit = (values ? (w - warps_qk) * per_v : w * per_k) + lane / L, piece = lane % L;
    const bool active = lane < (32 / L) * L && unit < (values ? p.G : n_qk);
    const int ch = (values ? n_qk * p.dk + unit * p.dv : unit * p.dk) + piece * 8;
    const int idx = n - p.q_start[req], slot = p.state_slots[req];
    constexpr int KEEP = TAPS - 1;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = 0.f;
    if (active) {
        const T* row = p.proj + (size_t)n * p.ld + p.col0 + ch;
        T* st = (KEEP > 0 && slot >= 0) ? p.state + (size_t)slot * KEEP * p.channels + ch : nullptr;
        Vec8<T> past[TAPS];                                 // past[b]: the projected values b positions back
        past[0].load(row);
#pragma unroll
        for (int b = 1; b < TAPS; ++b) {
            past[b].zero();
            if (pos - b >= 0) {
                if (idx - b >= 0) past[b].load(row - (ptrdiff_t)b * p.ld);
                else if (st) past[b].load(st + (size_t)(KEEP + idx - b) * p.channels);
            }
        }
        if (p.conv_w == nullptr) {
            past[0].get(y);
        } else {
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                float u[8];
                past[TAPS - 1 - j].get(u);
                const float4 w0 = *(const float4*)(p.conv_w + (size_t)j * p.channels + ch);
                const float4 w1 = *(const float4*)(p.conv_w + (size_t)j * p.channels + ch + 4);
                y[0] = fmaf(w0.x, u[0], y[0]); y[1] = fmaf(w0.y, u[1], y[1]); y[2] = fmaf(w0.z, u[2], y[2]); y[3] = fmaf(w0.w, u[3], y[3]);
                y[4] = fmaf(w1.x, u[4], y[4]); y[5] = fmaf(w1.y, u[5], y[5]); y[6] = fmaf(w1.z, u[6], y[6]); y[7] = fmaf(w1.w, u[7], y[7]);
            }
            if (st && p.q_len[req] == 1) {                  // oldest first: what was one back is now two back
#pragma unroll
                for (int s = 0; s < KEEP; ++s) past[KEEP - 1 - s].store(st + (size_t)s * p.channels);
            }
        }
    }
    const bool is_q = !values && unit < p.H;
    const float* g = values ? nullptr : (is_q ? p.q_norm : p.k_norm);
    if (!values) {
        float ssq = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ssq = fmaf(y[i], y[i], ssq);
        float total = 0.f;
        if ((L & (L - 1)) == 0) {                           // the head's lanes are an aligned power of two: a butterfly
            total = ssq;
            for (int o = L >> 1; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        } else {
            const int seg = (lane / L) * L;
            for (int o = 0; o < L; ++o) total += __shfl_sync(0xffffffffu, ssq, (seg + o) & 31);
        }
        if (active && g != nullptr) {
            const float rinv = 1.0f / sqrtf(total / (float)dims + p.eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] *= rinv * g[piece * 8 + i];
        }
        if (active && p.rot_dims > 0) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int c = piece * 8 + 2 * t;
                if (c + 1 < p.rot_dims) {
                    const float2 cs_sn = turn[c >> 1];
                    const float a = y[2 * t], b = y[2 * t + 1];
                    y[2 * t] = a * cs_sn.x - b * cs_sn.y;
                    y[2 * t + 1] = b * cs_sn.x + a * cs_sn.y;
                }
            }
        }
    }
    if (!active) return;
    T* out = values ? p.v_out + ((size_t)n * p.G + unit) * p.D
                    : (is_q ? p.q_out + ((size_t)n * p.H + unit) * p.D : p.k_out + ((size_t)n * p.G + (unit - p.H)) * p.D);
    Vec8<T> o;
    o.set(y);
    o.store(out + piece * 8);
    o.zero();
    for (int pp = L + piece; pp < (p.D >> 3); pp += L) o.store(out + pp * 8);       // the head's padding
}

// After a step: the state of every request with more than one row (q_len 1: the kernel above did it) becomes its last
// taps - 1 projected values.  A thread owns a channel and walks the state from the oldest entry on: what it reads
// (further on in the old state, or this step's rows) it has not yet overwritten.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, int ld, int col0, T* state, int keep, int channels,
                                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                                         const int* __restrict__ state_slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y;
    const int len = q_len[r], slot = state_slots[r];
    if (len <= 1 || slot < 0) return;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= channels) return;
    T* st = state + (size_t)slot * keep * channels + ch;
    const T* rows = proj + (size_t)q_start[r] * ld + col0 + ch;
    for (int s = 0; s < keep; ++s) {
        const int rel = len - keep + s;                     // which of this step's rows it is; negative: still the old state's
        st[(size_t)s * channels] = rel >= 0 ? rows[(size_t)rel * ld] : st[(size_t)(s + len) * channels];
    }
}

template <typename T>
int launch(const void* proj, int ld, int col0, const float* conv_w, int taps, void* state, const int* token_request,
           const int* positions, const int* q_start, const int* q_len, const int* state_slots, int n_requests,
           int update_state, const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rot_dims,
           int interleaved, float magnitude, void* q_out, void* k_out, void* v_out, int N, int H, int G, int dk, int dv,
           int D, cudaStream_t stream) {
    ConvPrep<T> p;
    p.proj = (const T*)proj; p.ld = ld; p.col0 = col0; p.conv_w = conv_w; p.taps = conv_w ? taps : 1; p.state = (T*)state;
    p.token_request = token_request; p.positions = positions; p.q_start = q_start; p.q_len = q_len;
    p.state_slots = state_slots; p.q_norm = q_norm; p.k_norm = k_norm; p.eps = eps; p.inv_freq = inv_freq;
    p.rot_dims = inv_freq ? rot_dims : 0; p.interleaved = interleaved; p.magnitude = magnitude;
    p.q_out = (T*)q_out; p.k_out = (T*)k_out; p.v_out = (T*)v_out; p.H = H; p.G = G; p.dk = dk; p.dv = dv; p.D = D;
    p.channels = H * dk + G * (dk + dv);
    // the vectorised kernel where the sizes and addresses allow 8-channel pieces
    const size_t el = sizeof(T);
    const bool vec = dk % 8 == 0 && (G == 0 || dv % 8 == 0) && D % 8 == 0 && (p.rot_dims == 0 || interleaved) && p.taps <= 4 &&
                     ld % 8 == 0 && col0 % 8 == 0 && ((uintptr_t)proj * 1) % 16 == 0 && ((uintptr_t)state % 16) == 0 &&
                     ((uintptr_t)conv_w % 16) == 0 && (((uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)v_out) % 16) == 0 && el >= 2;
    int rc;
    if (vec) {
        const int per_k = 32 / (dk / 8), per_v = G ? 32 / (dv / 8) : 1;
        const int warps = (H + G + per_k - 1) / per_k + (G ? (G + per_v - 1) / per_v : 0);
        const dim3 grid(N, (warps + 3) / 4);
        switch (p.taps) {
            case 1: rc = tnx_launch_in_order(conv_norm_rotate_vec_kernel<T, 1>, grid, dim3(128), 0, stream, p); break;
            case 2: rc = tnx_launch_in_order(conv_norm_rotate_vec_kernel<T, 2>, grid, dim3(128), 0, stream, p); break;
            case 3: rc = tnx_launch_in_order(conv_norm_rotate_vec_kernel<T, 3>, grid, dim3(128), 0, stream, p); break;
            default: rc = tnx_launch_in_order(conv_norm_rotate_vec_kernel<T, 4>, grid, dim3(128), 0, stream, p); break;
        }
    } else {
        rc = tnx_launch_in_order(conv_norm_rotate_kernel<T>, dim3(N), dim3(128), 0, stream, p);
    }
    if (rc != 0 || !update_state || p.taps <= 1 || n_requests <= 0) return rc;
    return tnx_launch_in_order(conv_state_update_kernel<T>, dim3((p.channels + 127) / 128, n_requests), dim3(128), 0, stream,
                               (const T*)proj, ld, col0, (T*)state, p.taps - 1, p.channels, q_start, q_len, state_slots);
}
}  // namespace

// update_state: 0 when every request of the step has one row (nothing is left for the second kernel).
TNX_EXPORT int tnx_conv_qkv_prep(const void* proj, int ld, int col0, const float* conv_w, int taps, void* state,
                                 const int* token_request, const int* positions, const int* q_start, const int* q_len,
                                 const int* state_slots, int n_requests, int update_state, const float* q_norm,
                                 const float* k_norm, float eps, const float* inv_freq, int rot_dims, int interleaved,
                                 float magnitude, void* q_out, void* k_out, void* v_out, int N, int H, int G, int dk, int dv,
                                 int D, int is_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || G < 0 || dk <= 0 || dv <= 0 || D < dk || D < dv || D > 64 * MAX_R || taps < 1 || taps > MAX_TAPS ||
        rot_dims < 0 || rot_dims % 2 || rot_dims > dk)
        return TNX_ERR_UNSUPPORTED;
    if (conv_w && taps > 1 && !state) return TNX_ERR_BAD_ARG;
    if (is_h16)
        return launch<h16>(proj, ld, col0, conv_w, taps, state, token_request, positions, q_start, q_len, state_slots,
                           n_requests, update_state, q_norm, k_norm, eps, inv_freq, rot_dims, interleaved, magnitude, q_out,
                           k_out, v_out, N, H, G, dk, dv, D, stream);
    return launch<float>(proj, ld, col0, conv_w, taps, state, token_request, positions, q_start, q_len, state_slots,
                         n_requests, update_state, q_norm, k_norm, eps, inv_freq, rot_dims, interleaved, magnitude, q_out,
                         k_out, v_out, N, H, G, dk, dv, D, stream);
}

// The state kernel alone, for another mixer whose own kernel does the convolution: the state [slots, keep, channels] of
// every request with more than one row becomes its last `keep` projected values (columns col0 .. col0 + channels of proj).
TNX_EXPORT int tnx_conv_state_update(const void* proj, int ld, int col0, void* state, int keep, int channels,
                                     const int* q_start, const int* q_len, const int* state_slots, int n_requests,
                                     int is_h16, cudaStream_t stream) {
    if (n_requests <= 0 || keep <= 0) return 0;
    if (channels <= 0 || !proj || !state) return TNX_ERR_BAD_ARG;
    const dim3 grid((channels + 127) / 128, n_requests);
    if (is_h16)
        return tnx_launch_in_order(conv_state_update_kernel<h16>, grid, dim3(128), 0, stream, (const h16*)proj, ld, col0,
                                   (h16*)state, keep, channels, q_start, q_len, state_slots);
    return tnx_launch_in_order(conv_state_update_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, ld, col0,
                               (float*)state, keep, channels, q_start, q_len, state_slots);
}
