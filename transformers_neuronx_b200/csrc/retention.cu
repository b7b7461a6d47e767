// Retention: linear attention with a fixed decay per head, no softmax and no denominator.  Per head, with
// q_t, k_t of k_dim numbers and v_t of v_dim numbers:
//     S_t = decay * S_(t-1) + k_t v_t^T          (S: k_dim x v_dim, 32-bit, kept per request between steps)
//     o_t = S_t^T q_t
// Everything that enters the recurrence is 32-bit: queries and keys are rotated by position in 32-bit from the
// projection's output (tnx_retention_prep) and are not rounded again; the state lives in 32-bit.
//
// tnx_retention_prep: on the first rot_dims dims of each head, dim i paired with i + rot_dims/2, the pair
//   (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i]; keys are then
//   multiplied by k_scale.  Output: 32-bit q and k, [tokens, heads * k_dim].
// tnx_retention_scan: a thread block owns C columns (value dims) of one head of one request and walks the
//   request's tokens of this step in order, the state's columns in registers: a column's k_dim rows are spread
//   over R adjacent lanes, which add their partial sums of o_t with shuffles.  The state is stored
//   [slot, head, v_dim, k_dim] (a column's rows side by side), so that the R lanes of a column read one
//   contiguous piece.  A step of one token per request streams the state through once; a portion of a prompt
//   keeps it in registers for all its tokens.  Queries and keys of a few tokens at a time are staged in shared memory.
// tnx_headwise_gated_rms_norm: o of each (token, head) divided by its root mean square (eps inside the root,
//   an optional weight over the head's dims), multiplied by act(gate) (silu here; the activation is a parameter) and
//   by out_scale, written in the activation type.
#include "common.cuh"

namespace {

template <typename T>
__global__ void retention_prep_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off,
                                      const int* __restrict__ token_request, const int* __restrict__ positions,
                                      const float* __restrict__ inv_freq, int rot_dims, float k_scale,
                                      float* __restrict__ q_out, float* __restrict__ k_out, int H, int dk) {
    extern __shared__ float sm[];                   // cos and sin of the token's angles, the same for every head
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    if (token_request[n] < 0) return;
    const float pos = (float)positions[n];
    const T* row = proj + (size_t)n * ld;
    const int half = rot_dims / 2;
    float* cst = sm;
    float* snt = sm + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &snt[i], &cst[i]);
    __syncthreads();
    float* qd = q_out + (size_t)n * H * dk;
    float* kd = k_out + (size_t)n * H * dk;
    for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
        const int h = e / half, i = e % half;
        const int c0 = h * dk + i, c1 = c0 + half;
        const float sn = snt[i], cs = cst[i];
        const float qu = to_float(row[q_off + c0]), qv = to_float(row[q_off + c1]);
        const float ku = to_float(row[k_off + c0]), kv = to_float(row[k_off + c1]);
        qd[c0] = qu * cs - qv * sn;
        qd[c1] = qv * cs + qu * sn;
        kd[c0] = (ku * cs - kv * sn) * k_scale;
        kd[c1] = (kv * cs + ku * sn) * k_scale;
    }
    const int rest = dk - rot_dims;
    for (int e = threadIdx.x; e < H * rest; e += blockDim.x) {
        const int c = (e / rest) * dk + rot_dims + e % rest;
        qd[c] = to_float(row[q_off + c]);
        kd[c] = to_float(row[k_off + c]) * k_scale;
    }
}

constexpr int SCAN_TOKENS_MOST = 32;  // most tokens whose queries and keys are staged in shared memory at a time
constexpr int SCAN_STAGES = 2;        // one stage is computed on while the next one arrives

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// What may change from token to token (a selective state-space recurrence): S_t = decay_t S_(t-1) + kscale_t k_t v_t^T with
// decay [tokens, H] and kscale [tokens, H] (each absent: the head's fixed decay, 1), and queries and keys that the heads
// of a group share: qk_heads of them for H heads, head h reading those of h / (H / qk_heads).  A stage carries its
// tokens' two numbers behind its values.
struct TokenGates {
    const float* decay;
    const float* kscale;
    int qk_heads;
};
__host__ __device__ __forceinline__ int token_gate_floats(int stage_tokens) { return (2 * stage_tokens + 3) & ~3; }

// KPT: rows of a column one thread keeps; R: lanes a column's rows are spread over (KPT * R >= k_dim).
// VEC: k_dim is a multiple of four: a thread's rows come in runs of four (rows 4 (r + R m) .. + 3), read as one
// 16-byte piece, and the stages are filled with 16-byte asynchronous copies; otherwise with plain loads.
// VASYNC: the values' rows of the block's columns are whole 16-byte pieces too and are staged the same way, in the
// type they are stored in (converted where they are used); otherwise plain loads convert them on the way in.
// The R partial sums of an output are not added with shuffles token by token (a chain of round trips that the few
// warps of a block cannot hide): every thread leaves its partial sum in shared memory, and after a stage's tokens
// the block adds them up and stores the outputs.
// A stage holds q [ST][DKP], k [ST][DKP] (columns from k_dim on stay zero) and v [ST][C], ST = stage_tokens: 32 for
// portions of prompts, as few as one for a step of single tokens (less shared memory, more blocks an SM).
template <typename T, int KPT, int R, bool VEC, bool VASYNC>
__global__ void __launch_bounds__(16 * R < 128 ? 128 : 16 * R)
retention_scan_kernel(const float* __restrict__ qr, const float* __restrict__ kr, const T* __restrict__ v, int v_ld,
                      const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ q_start,
                      const int* __restrict__ q_len, const int* __restrict__ state_slots, float* __restrict__ out,
                      int H, int dk, int dv, int C, int stage_tokens, TokenGates tg) {
    constexpr int DKP = KPT * R;
    const int SCAN_TOKENS = stage_tokens;
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.z, h = blockIdx.y;
    const int len = q_len[req];
    if (len <= 0) return;                            // a padded request of a captured batch
    const int slot = state_slots[req];
    if (slot < 0) return;
    const int t_first = q_start[req];
    const int stage_floats = SCAN_TOKENS * (2 * DKP + C) + token_gate_floats(SCAN_TOKENS);
    float* part = sm + SCAN_STAGES * stage_floats;    // [SCAN_TOKENS][C * R] partial sums of the stage being computed
    const int jl = threadIdx.x / R, r = threadIdx.x % R;
    const int j = blockIdx.x * C + jl;
    const bool col = j < dv;
    const float dec_fixed = decay ? decay[h] : 1.f;
    const int Hq = tg.qk_heads, hq = h / (H / Hq);
    float* st = state + (((size_t)slot * H + h) * dv + (col ? j : 0)) * dk;

    // Fills stage `s` with the tokens from t0 on: queries and keys by asynchronous copies (VEC) or plain loads,
    // values by asynchronous copies in their stored type (VASYNC) or by plain loads that convert them.
    auto fill = [&](int s, int t0) {
        float* qs = sm + s * stage_floats;
        float* ks = qs + SCAN_TOKENS * DKP;
        float* vs = ks + SCAN_TOKENS * DKP;
        const int nt = min(SCAN_TOKENS, len - t0);
        const size_t g0 = (size_t)(t_first + t0) * Hq * dk + (size_t)hq * dk;
        if (VEC) {
            const int pieces = dk / 4;
            for (int e = threadIdx.x; e < nt * pieces; e += blockDim.x) {
                const int tt = e / pieces, c = e % pieces;
                cp_async_16(qs + tt * DKP + 4 * c, qr + g0 + (size_t)tt * Hq * dk + 4 * c);
                cp_async_16(ks + tt * DKP + 4 * c, kr + g0 + (size_t)tt * Hq * dk + 4 * c);
            }
        } else {
            for (int e = threadIdx.x; e < nt * dk; e += blockDim.x) {
                const int tt = e / dk, i = e % dk;
                qs[tt * DKP + i] = qr[g0 + (size_t)tt * Hq * dk + i];
                ks[tt * DKP + i] = kr[g0 + (size_t)tt * Hq * dk + i];
            }
        }
        float* gs = vs + SCAN_TOKENS * C;              // [decay of the stage's tokens][their key scales]
        for (int e = threadIdx.x; e < nt; e += blockDim.x) {
            const size_t at = (size_t)(t_first + t0 + e) * H + h;
            gs[e] = tg.decay ? tg.decay[at] : dec_fixed;
            gs[SCAN_TOKENS + e] = tg.kscale ? tg.kscale[at] : 1.f;
        }
        if (VASYNC) {
            constexpr int PER = 16 / sizeof(T);       // values in a 16-byte piece
            const int vp = C / PER;
            T* vraw = (T*)vs;
            for (int e = threadIdx.x; e < nt * vp; e += blockDim.x) {
                const int tt = e / vp, c = e % vp;
                cp_async_16(vraw + tt * C + PER * c,
                            v + (size_t)(t_first + t0 + tt) * v_ld + (size_t)h * dv + blockIdx.x * C + PER * c);
            }
        }
        cp_async_commit();
        if (!VASYNC) {
            for (int e = threadIdx.x; e < nt * C; e += blockDim.x) {
                const int tt = e / C, c = blockIdx.x * C + e % C;
                vs[e] = c < dv ? to_float(v[(size_t)(t_first + t0 + tt) * v_ld + (size_t)h * dv + c]) : 0.f;
            }
        }
    };

    if (DKP > dk) {                                  // the rows' padding is zeroed once and never written again
        const int pad = DKP - dk;
        for (int e = threadIdx.x; e < SCAN_STAGES * 2 * SCAN_TOKENS * pad; e += blockDim.x) {
            const int rowi = e / pad, c = dk + e % pad;
            const int s = rowi / (2 * SCAN_TOKENS), within = rowi % (2 * SCAN_TOKENS);
            sm[s * stage_floats + within * DKP + c] = 0.f;
        }
    }
    fill(0, 0);
    float S[KPT];
    if (VEC) {
#pragma unroll
        for (int m4 = 0; m4 < KPT / 4; ++m4) {
            const int i = 4 * (r + R * m4);
            const float4 s4 = (col && i < dk) ? *(const float4*)(st + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            S[4 * m4 + 0] = s4.x; S[4 * m4 + 1] = s4.y; S[4 * m4 + 2] = s4.z; S[4 * m4 + 3] = s4.w;
        }
    } else {
#pragma unroll
        for (int m = 0; m < KPT; ++m) S[m] = (col && r + R * m < dk) ? st[r + R * m] : 0.f;
    }
    int stage = 0;
    for (int t0 = 0; t0 < len; t0 += SCAN_TOKENS, stage ^= 1) {
        const int nt = min(SCAN_TOKENS, len - t0);
        cp_async_wait_all();
        __syncthreads();                              // this stage has arrived; the other one is no longer read
        if (t0 + SCAN_TOKENS < len) fill(stage ^ 1, t0 + SCAN_TOKENS);
        const float* qs = sm + stage * stage_floats;
        const float* ks = qs + SCAN_TOKENS * DKP;
        const float* vs = ks + SCAN_TOKENS * DKP;
        const float* gs = vs + SCAN_TOKENS * C;
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {
            const float dec = gs[tt];
            const float vj = (VASYNC ? to_float(((const T*)vs)[tt * C + jl]) : vs[tt * C + jl]) * gs[SCAN_TOKENS + tt];
            const float* kt = ks + tt * DKP;
            const float* qt = qs + tt * DKP;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            if (VEC) {
#pragma unroll
                for (int m4 = 0; m4 < KPT / 4; ++m4) {
                    const float4 k4 = ((const float4*)kt)[r + R * m4];
                    const float4 q4 = ((const float4*)qt)[r + R * m4];
                    S[4 * m4 + 0] = fmaf(dec, S[4 * m4 + 0], k4.x * vj); a0 = fmaf(S[4 * m4 + 0], q4.x, a0);
                    S[4 * m4 + 1] = fmaf(dec, S[4 * m4 + 1], k4.y * vj); a1 = fmaf(S[4 * m4 + 1], q4.y, a1);
                    S[4 * m4 + 2] = fmaf(dec, S[4 * m4 + 2], k4.z * vj); a2 = fmaf(S[4 * m4 + 2], q4.z, a2);
                    S[4 * m4 + 3] = fmaf(dec, S[4 * m4 + 3], k4.w * vj); a3 = fmaf(S[4 * m4 + 3], q4.w, a3);
                }
            } else {
#pragma unroll
                for (int m = 0; m < KPT; ++m) {
                    S[m] = fmaf(dec, S[m], kt[r + R * m] * vj);
                    if (m & 1) a1 = fmaf(S[m], qt[r + R * m], a1); else a0 = fmaf(S[m], qt[r + R * m], a0);
                }
            }
            part[tt * (C * R) + threadIdx.x] = (a0 + a1) + (a2 + a3);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nt * C; e += blockDim.x) {
            const int tt = e / C, c = e % C;
            const float* p = part + tt * (C * R) + c * R;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) acc += p[i];
            if (blockIdx.x * C + c < dv) out[(size_t)(t_first + t0 + tt) * H * dv + (size_t)h * dv + blockIdx.x * C + c] = acc;
        }
    }
    if (col) {
        if (VEC) {
#pragma unroll
            for (int m4 = 0; m4 < KPT / 4; ++m4) {
                const int i = 4 * (r + R * m4);
                if (i < dk) *(float4*)(st + i) = make_float4(S[4 * m4 + 0], S[4 * m4 + 1], S[4 * m4 + 2], S[4 * m4 + 3]);
            }
        } else {
#pragma unroll
            for (int m = 0; m < KPT; ++m)
                if (r + R * m < dk) st[r + R * m] = S[m];
        }
    }
}

// The form for a step of single tokens (key sizes that are multiples of four).  A thread keeps FOUR columns' rows, so
// a block streams 4 x as much of the state with the same staging, and every key and query value it reads from shared
// memory feeds four columns.  Thread (g, r) of a block: columns 4g .. 4g+3 of the
// block's C, rows 4 (r + R m) .. + 3 for m < KPT/4.  Partial sums go to shared memory as [token][g][r][4] (a group of R
// pieces padded by one piece, so that the adding pass meets no bank twice), and are added after the stage's tokens.
template <typename T, int KPT, int R>
__global__ void __launch_bounds__(128)
retention_scan4_kernel(const float* __restrict__ qr, const float* __restrict__ kr, const T* __restrict__ v, int v_ld,
                       const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ q_start,
                       const int* __restrict__ q_len, const int* __restrict__ state_slots, float* __restrict__ out,
                       int H, int dk, int dv, int C, int stage_tokens, TokenGates tg) {
    constexpr int DKP = KPT * R;
    constexpr int GROUP = 4 * R + 4;                 // floats of one (token, column group) in `part`
    const int ST = stage_tokens, CG = C / 4;
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.z, h = blockIdx.y;
    const int len = q_len[req];
    if (len <= 0) return;                            // a padded request of a captured batch
    const int slot = state_slots[req];
    if (slot < 0) return;
    const int t_first = q_start[req];
    const int stage_floats = ST * (2 * DKP + C) + token_gate_floats(ST);
    float* part = sm + SCAN_STAGES * stage_floats;   // [ST][CG][GROUP]
    const int g = threadIdx.x / R, r = threadIdx.x % R;
    const int j0 = blockIdx.x * C + 4 * g;
    const float dec_fixed = decay ? decay[h] : 1.f;
    const int Hq = tg.qk_heads, hq = h / (H / Hq);
    float* st = state + (((size_t)slot * H + h) * dv) * dk;

    auto fill = [&](int s, int t0) {
        float* qs = sm + s * stage_floats;
        float* ks = qs + ST * DKP;
        float* vs = ks + ST * DKP;
        const int nt = min(ST, len - t0);
        const size_t g0 = (size_t)(t_first + t0) * Hq * dk + (size_t)hq * dk;
        const int pieces = dk / 4;
        for (int e = threadIdx.x; e < nt * pieces; e += blockDim.x) {
            const int tt = e / pieces, c = e % pieces;
            cp_async_16(qs + tt * DKP + 4 * c, qr + g0 + (size_t)tt * Hq * dk + 4 * c);
            cp_async_16(ks + tt * DKP + 4 * c, kr + g0 + (size_t)tt * Hq * dk + 4 * c);
        }
        cp_async_commit();
        float* gs = vs + ST * C;
        for (int e = threadIdx.x; e < nt; e += blockDim.x) {
            const size_t at = (size_t)(t_first + t0 + e) * H + h;
            gs[e] = tg.decay ? tg.decay[at] : dec_fixed;
            gs[ST + e] = tg.kscale ? tg.kscale[at] : 1.f;
        }
        for (int e = threadIdx.x; e < nt * C; e += blockDim.x) {
            const int tt = e / C, c = blockIdx.x * C + e % C;
            vs[e] = c < dv ? to_float(v[(size_t)(t_first + t0 + tt) * v_ld + (size_t)h * dv + c]) : 0.f;
        }
    };

    if (DKP > dk) {                                  // the rows' padding is zeroed once and never written again
        const int pad = DKP - dk;
        for (int e = threadIdx.x; e < SCAN_STAGES * 2 * ST * pad; e += blockDim.x) {
            const int rowi = e / pad, c = dk + e % pad;
            sm[(rowi / (2 * ST)) * stage_floats + (rowi % (2 * ST)) * DKP + c] = 0.f;
        }
    }
    fill(0, 0);
    float S[4][KPT];
#pragma unroll
    for (int ct = 0; ct < 4; ++ct)
#pragma unroll
        for (int m4 = 0; m4 < KPT / 4; ++m4) {
            const int i = 4 * (r + R * m4);
            const float4 s4 = (j0 + ct < dv && i < dk) ? *(const float4*)(st + (size_t)(j0 + ct) * dk + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            S[ct][4 * m4 + 0] = s4.x; S[ct][4 * m4 + 1] = s4.y; S[ct][4 * m4 + 2] = s4.z; S[ct][4 * m4 + 3] = s4.w;
        }
    int stage = 0;
    for (int t0 = 0; t0 < len; t0 += ST, stage ^= 1) {
        const int nt = min(ST, len - t0);
        cp_async_wait_all();
        __syncthreads();                              // this stage has arrived; the other one and `part` are no longer read
        if (t0 + ST < len) fill(stage ^ 1, t0 + ST);
        const float* qs = sm + stage * stage_floats;
        const float* ks = qs + ST * DKP;
        const float* vs = ks + ST * DKP;
        const float* gs = vs + ST * C;
        for (int tt = 0; tt < nt; ++tt) {
            const float4 v4 = *(const float4*)(vs + tt * C + 4 * g);
            const float dec = gs[tt], ksc = gs[ST + tt];
            const float vj[4] = {v4.x * ksc, v4.y * ksc, v4.z * ksc, v4.w * ksc};
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m4 = 0; m4 < KPT / 4; ++m4) {
                const float4 k4 = ((const float4*)(ks + tt * DKP))[r + R * m4];
                const float4 q4 = ((const float4*)(qs + tt * DKP))[r + R * m4];
                const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int ct = 0; ct < 4; ++ct)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        S[ct][4 * m4 + e] = fmaf(dec, S[ct][4 * m4 + e], kk[e] * vj[ct]);
                        acc[ct] = fmaf(S[ct][4 * m4 + e], qq[e], acc[ct]);
                    }
            }
            *(float4*)(part + (tt * CG + g) * GROUP + 4 * r) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nt * C; e += blockDim.x) {
            const int grp = e / 4, ct = e % 4;            // grp = tt * CG + g
            const float* p = part + grp * GROUP + ct;
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) a += p[4 * i];
            const int tt = grp / CG, j = blockIdx.x * C + 4 * (grp % CG) + ct;
            if (j < dv) out[(size_t)(t_first + t0 + tt) * H * dv + (size_t)h * dv + j] = a;
        }
    }
#pragma unroll
    for (int ct = 0; ct < 4; ++ct)
#pragma unroll
        for (int m4 = 0; m4 < KPT / 4; ++m4) {
            const int i = 4 * (r + R * m4);
            if (j0 + ct < dv && i < dk)
                *(float4*)(st + (size_t)(j0 + ct) * dk + i) = make_float4(S[ct][4 * m4 + 0], S[ct][4 * m4 + 1], S[ct][4 * m4 + 2], S[ct][4 * m4 + 3]);
        }
}

// A step of single tokens in ONE kernel (key and value sizes that are multiples of four): what retention_prep, the scan
// and the head-wise norm do, for one (request, head) a block, without the 32-bit q, k and o passing through memory.
// The block rotates its head's query and key of the request's token into shared memory (k scaled), streams the head's
// state through registers once (thread (g, r): columns 4g .. 4g+3, rows 4 (r + R m) .. + 3), adds the partial sums of
// o through shared memory, and then divides o by its root mean square, applies the gate and the scale and stores
// the activations.  Requests with no row are skipped; the caller uses it only where every request has one row.
template <typename T, int KPT, int R>
__global__ void __launch_bounds__(512)
retention_decode_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int g_off,
                        const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dims,
                        float k_scale, const float* __restrict__ decay, float* __restrict__ state,
                        const int* __restrict__ q_start, const int* __restrict__ q_len,
                        const int* __restrict__ state_slots, float eps, float out_scale, T* __restrict__ out, int out_ld,
                        int H, int dk, int dv) {
    constexpr int DKP = KPT * R;
    constexpr int GROUP = 4 * R + 4;
    extern __shared__ __align__(16) float sm[];      // q [DKP], k [DKP], v [dv4], gate [dv4], part [CG][GROUP], o [dv4]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.y, h = blockIdx.x;
    if (q_len[req] <= 0) return;                     // a padded request of a captured batch
    const int slot = state_slots[req];
    if (slot < 0) return;
    const int n = q_start[req];
    const int CG = (dv + 3) / 4, dv4 = 4 * CG;
    float* qs = sm;
    float* ks = qs + DKP;
    float* vs = ks + DKP;
    float* gs = vs + dv4;
    float* part = gs + dv4;
    float* os = part + CG * GROUP;
    const T* row = proj + (size_t)n * ld;
    const float pos = (float)positions[n];
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < DKP; i += blockDim.x) {
        float qv = 0.f, kv = 0.f;
        if (i < dk) {
            const int c = h * dk + i;
            qv = to_float(row[q_off + c]);
            kv = to_float(row[k_off + c]);
            if (i < rot_dims) {
                const int fi = i < half ? i : i - half;
                float sn, cs;
                sincosf(pos * inv_freq[fi], &sn, &cs);
                const int partner = i < half ? c + half : c - half;
                const float q2 = to_float(row[q_off + partner]), k2 = to_float(row[k_off + partner]);
                // the pair (u, v) becomes (u cos - v sin, v cos + u sin)
                qv = i < half ? qv * cs - q2 * sn : qv * cs + q2 * sn;
                kv = i < half ? kv * cs - k2 * sn : kv * cs + k2 * sn;
            }
            kv *= k_scale;
        }
        qs[i] = qv;
        ks[i] = kv;
    }
    for (int j = threadIdx.x; j < dv4; j += blockDim.x) {
        vs[j] = j < dv ? to_float(row[v_off + h * dv + j]) : 0.f;
        gs[j] = (j < dv && g_off >= 0) ? to_float(row[g_off + h * dv + j]) : 0.f;
    }
    __syncthreads();
    const int g = threadIdx.x / R, r = threadIdx.x % R;
    const float dec = decay[h];
    float* st = state + (((size_t)slot * H + h) * dv) * dk;
    if (g < CG) {
        const float4 v4 = *(const float4*)(vs + 4 * g);
        const float vj[4] = {v4.x, v4.y, v4.z, v4.w};
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        float4 S[4][KPT / 4];
        // every piece of the state this thread owns is asked for before the first one is used
#pragma unroll
        for (int ct = 0; ct < 4; ++ct)
#pragma unroll
            for (int m4 = 0; m4 < KPT / 4; ++m4) {
                const int i = 4 * (r + R * m4);
                S[ct][m4] = (4 * g + ct < dv && i < dk) ? *(const float4*)(st + (size_t)(4 * g + ct) * dk + i)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
        for (int m4 = 0; m4 < KPT / 4; ++m4) {
            const int i = 4 * (r + R * m4);            // rows beyond k_dim read the zero padding of q and k
            const float4 k4 = *(const float4*)(ks + i), q4 = *(const float4*)(qs + i);
#pragma unroll
            for (int ct = 0; ct < 4; ++ct) {
                float4& s4 = S[ct][m4];
                s4.x = fmaf(dec, s4.x, k4.x * vj[ct]); acc[ct] = fmaf(s4.x, q4.x, acc[ct]);
                s4.y = fmaf(dec, s4.y, k4.y * vj[ct]); acc[ct] = fmaf(s4.y, q4.y, acc[ct]);
                s4.z = fmaf(dec, s4.z, k4.z * vj[ct]); acc[ct] = fmaf(s4.z, q4.z, acc[ct]);
                s4.w = fmaf(dec, s4.w, k4.w * vj[ct]); acc[ct] = fmaf(s4.w, q4.w, acc[ct]);
            }
        }
#pragma unroll
        for (int ct = 0; ct < 4; ++ct)
#pragma unroll
            for (int m4 = 0; m4 < KPT / 4; ++m4) {
                const int i = 4 * (r + R * m4);
                if (4 * g + ct < dv && i < dk) *(float4*)(st + (size_t)(4 * g + ct) * dk + i) = S[ct][m4];
            }
        *(float4*)(part + g * GROUP + 4 * r) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
    __syncthreads();
    float ss = 0.f;
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
        const float* p = part + (j / 4) * GROUP + (j % 4);
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) a += p[4 * i];
        os[j] = a;
        ss += a * a;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)dv + eps);
    T* dst = out + (size_t)n * out_ld + (size_t)h * dv;
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
        float y = os[j] * rinv;
        if (g_off >= 0) { const float z = gs[j]; y *= z / (1.f + expf(-z)); }
        dst[j] = from_float<T>(y * out_scale);
    }
}

template <typename T>
__global__ void headwise_gated_rms_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_ld,
                                               const int* __restrict__ token_request, const float* __restrict__ w,
                                               float eps, float out_scale, T* __restrict__ out, int out_ld,
                                               int n_tokens, int H, int dv, int gate_act) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (pair >= (long long)n_tokens * H) return;
    const int n = (int)(pair / H), h = (int)(pair % H);
    if (token_request[n] < 0) return;
    const float* src = o + ((size_t)n * H + h) * dv;
    const T* g = gate ? gate + (size_t)n * gate_ld + (size_t)h * dv : nullptr;
    T* dst = out + (size_t)n * out_ld + (size_t)h * dv;
    if (dv % 4 == 0 && dv <= 512 && ((uintptr_t)src % 16) == 0) {
        // up to four runs of four values a lane, held in registers between the two passes
        float4 v[4];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = 4 * (lane + 32 * i);
            v[i] = c < dv ? *(const float4*)(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
        }
        s = warp_sum(s);
        const float rinv = 1.0f / sqrtf(s / (float)dv + eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = 4 * (lane + 32 * i);
            if (c >= dv) continue;
            float y[4] = {v[i].x * rinv, v[i].y * rinv, v[i].z * rinv, v[i].w * rinv};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (w) y[e] *= w[c + e];
                if (g) y[e] *= apply_activation(to_float(g[c + e]), gate_act);
                dst[c + e] = from_float<T>(y[e] * out_scale);
            }
        }
        return;
    }
    float s = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = src[c]; s += v * v; }
    s = warp_sum(s);
    const float rinv = 1.0f / sqrtf(s / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        float y = src[c] * rinv;
        if (w) y *= w[c];
        if (g) y *= apply_activation(to_float(g[c]), gate_act);
        dst[c] = from_float<T>(y * out_scale);
    }
}

}  // namespace

TNX_EXPORT int tnx_retention_prep(const void* proj, int ld, int q_off, int k_off, const int* token_request,
                                  const int* positions, const float* inv_freq, int rot_dims, float k_scale, float* q_out,
                                  float* k_out, int n_tokens, int H, int dk, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || dk <= 0 || rot_dims < 0 || rot_dims > dk || rot_dims % 2 || (rot_dims && !inv_freq)) return TNX_ERR_BAD_ARG;
    const int threads = H * dk >= 2048 ? 256 : 128;
    const size_t smem = (size_t)rot_dims * sizeof(float);
    if (is_h16)
        return tnx_launch_in_order(retention_prep_kernel<h16>, dim3(n_tokens), dim3(threads), smem, stream, (const h16*)proj, ld,
                                   q_off, k_off, token_request, positions, inv_freq, rot_dims, k_scale, q_out, k_out, H, dk);
    return tnx_launch_in_order(retention_prep_kernel<float>, dim3(n_tokens), dim3(threads), smem, stream, (const float*)proj, ld,
                               q_off, k_off, token_request, positions, inv_freq, rot_dims, k_scale, q_out, k_out, H, dk);
}

// The columns a thread block of the scan owns: 16 (8 where the head has fewer; columns beyond the head are
// idle lanes), so that even one request of a few heads spreads over many SMs and every block is whole warps.
TNX_EXPORT int tnx_retention_scan_columns(int dv) { return dv >= 16 ? 16 : 8; }

static int g_force_lanes = 0, g_force_stage = 0;

template <typename T>
static int retention_scan_launch(const float* qr, const float* kr, const T* v, int v_ld, const float* decay, float* state,
                                 const int* q_start, const int* q_len, const int* state_slots, float* out, int n_requests,
                                 int H, int dk, int dv, int stage_tokens, TokenGates tg, cudaStream_t stream) {
    const int C = tnx_retention_scan_columns(dv);
    const dim3 grid((dv + C - 1) / C, H, n_requests);
    const bool vec = dk % 4 == 0 && ((uintptr_t)qr % 16) == 0 && ((uintptr_t)kr % 16) == 0 && ((uintptr_t)state % 16) == 0;
    const bool vasync = dv % C == 0 && (C * sizeof(T)) % 16 == 0 && ((uintptr_t)v % 16) == 0 && ((size_t)v_ld * sizeof(T)) % 16 == 0 &&
                        ((size_t)dv * sizeof(T)) % 16 == 0;
#define SCAN(KPT, R)                                                                                                    \
    do {                                                                                                                \
        const size_t smem = ((size_t)SCAN_STAGES * (stage_tokens * (2 * (KPT) * (R) + C) + token_gate_floats(stage_tokens)) + (size_t)stage_tokens * C * (R)) * sizeof(float); \
        if (vec && vasync) {                                                                                            \
            if (smem > 48 * 1024)                                                                                       \
                cudaFuncSetAttribute(retention_scan_kernel<T, KPT, R, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            return tnx_launch_in_order(retention_scan_kernel<T, KPT, R, true, true>, grid, dim3(C * (R)), smem, stream, \
                                       qr, kr, v, v_ld, decay, state, q_start, q_len, state_slots, out, H, dk, dv, C,   \
                                       stage_tokens, tg);                                                               \
        }                                                                                                               \
        if (vec) {                                                                                                      \
            if (smem > 48 * 1024)                                                                                       \
                cudaFuncSetAttribute(retention_scan_kernel<T, KPT, R, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            return tnx_launch_in_order(retention_scan_kernel<T, KPT, R, true, false>, grid, dim3(C * (R)), smem, stream, \
                                       qr, kr, v, v_ld, decay, state, q_start, q_len, state_slots, out, H, dk, dv, C,   \
                                       stage_tokens, tg);                                                               \
        }                                                                                                               \
        if (smem > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(retention_scan_kernel<T, KPT, R, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tnx_launch_in_order(retention_scan_kernel<T, KPT, R, false, false>, grid, dim3(C * (R)), smem, stream, qr, kr, \
                                   v, v_ld, decay, state, q_start, q_len, state_slots, out, H, dk, dv, C, stage_tokens, tg); \
    } while (0)
#define SCAN4(KPT, R, CC)                                                                                               \
    do {                                                                                                                \
        const int C4 = (CC);                                                                                            \
        const dim3 grid4((dv + C4 - 1) / C4, H, n_requests);                                                            \
        const size_t smem = ((size_t)SCAN_STAGES * (stage_tokens * (2 * (KPT) * (R) + C4) + token_gate_floats(stage_tokens)) + \
                             (size_t)stage_tokens * (C4 / 4) * (4 * (R) + 4)) * sizeof(float);                          \
        if (smem > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(retention_scan4_kernel<T, KPT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tnx_launch_in_order(retention_scan4_kernel<T, KPT, R>, grid4, dim3((C4 / 4) * (R)), smem, stream, qr,    \
                                   kr, v, v_ld, decay, state, q_start, q_len, state_slots, out, H, dk, dv, C4,          \
                                   stage_tokens, tg);                                                                   \
    } while (0)
    // Measured (32 heads of 128 x 128): a step of single tokens streams the state at 6.2 TB/s in the four-column form
    // (43 us for 64 requests); portions of prompts are a chain of dependent tokens in either form, and there the
    // one-column form, with twice the warps, is the faster one (0.58 against 0.73 ms for 2,048 tokens).
    if (vec && stage_tokens == 1) {
        if (dk <= 16) SCAN4(4, 4, 32);
        if (dk <= 32) SCAN4(4, 8, 16);
        if (dk <= 64) SCAN4(4, 16, 16);
        if (dk <= 128) SCAN4(8, 16, 16);
        if (dk <= 256) SCAN4(16, 16, 16);
        return TNX_ERR_UNSUPPORTED;
    }
#undef SCAN4
    if (dk <= 16) SCAN(4, 4);
    if (dk <= 32) SCAN(4, 8);
    if (dk <= 64) SCAN(8, 8);
    if (dk <= 128) { if (g_force_lanes == 16) SCAN(8, 16); SCAN(16, 8); }
    if (dk <= 256) SCAN(32, 8);
    return TNX_ERR_UNSUPPORTED;
#undef SCAN
}

// A test and measurement hook: the lanes a column's rows are spread over (0: the kernel's own choice; 16 for key sizes
// of 65 to 128) and the most tokens of a stage (0: SCAN_TOKENS_MOST).
TNX_EXPORT int tnx_retention_scan_force(int lanes, int stage_tokens) {
    if ((lanes != 0 && lanes != 16) || stage_tokens < 0 || stage_tokens > SCAN_TOKENS_MOST) return TNX_ERR_BAD_ARG;
    g_force_lanes = lanes;
    g_force_stage = stage_tokens;
    return 0;
}

TNX_EXPORT int tnx_retention_scan(const float* qr, const float* kr, const void* v, int v_ld, const float* decay,
                                  float* state, const int* q_start, const int* q_len, const int* state_slots, float* out,
                                  int n_requests, int H, int dk, int dv, int most_tokens, int v_h16,
                                  const float* decay_tok, const float* kscale_tok, int qk_heads, cudaStream_t stream) {
    // most_tokens: an upper bound of the requests' rows (1 for a step of single tokens); it sizes the stages.
    // decay_tok, kscale_tok [tokens, H]: a decay and a key scale per token (absent: decay[h], 1); qk_heads: how many
    // heads q and k have (H, or fewer when groups of heads share them).
    if (n_requests <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || n_requests > 65535 || most_tokens <= 0) return TNX_ERR_BAD_ARG;
    if (qk_heads <= 0 || H % qk_heads || (!decay && !decay_tok)) return TNX_ERR_BAD_ARG;
    const TokenGates tg{decay_tok, kscale_tok, qk_heads};
    int stage_tokens = 1;
    int stage_most = g_force_stage ? g_force_stage : SCAN_TOKENS_MOST;
    if (!g_force_stage && dk > 64) {
        // Stages of 32 tokens of 128-row keys and queries take 86 KB, so an SM holds two blocks.  With more blocks than
        // that, smaller stages (more blocks at once, a rendezvous more often) are faster.  Measured at 128 rows and 64
        // columns a head, 2,048 tokens: 256 blocks 471 / 499 / 564 us with 32 / 16 / 8 tokens a stage, 512 blocks 920 / 793 /
        // 855, 2,048 blocks (eight requests of 256 tokens) 424 / 368 / 354.
        static int sms = 0;
        if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); if (sms <= 0) sms = 1; }
        const int C = tnx_retention_scan_columns(dv);
        const long long blocks = (long long)((dv + C - 1) / C) * H * n_requests;
        stage_most = blocks <= 2LL * sms ? 32 : (blocks <= 8LL * sms ? 16 : 8);
    }
    while (stage_tokens < most_tokens && stage_tokens < stage_most) stage_tokens *= 2;
    if (v_h16)
        return retention_scan_launch<h16>(qr, kr, (const h16*)v, v_ld, decay, state, q_start, q_len, state_slots, out,
                                          n_requests, H, dk, dv, stage_tokens, tg, stream);
    return retention_scan_launch<float>(qr, kr, (const float*)v, v_ld, decay, state, q_start, q_len, state_slots, out,
                                        n_requests, H, dk, dv, stage_tokens, tg, stream);
}

TNX_EXPORT int tnx_headwise_gated_rms_norm(const float* o, const void* gate, int gate_ld, const int* token_request,
                                           const float* w, float eps, float out_scale, void* out, int out_ld,
                                           int n_tokens, int H, int dv, int gate_act, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || dv <= 0 || out_ld < H * dv || gate_act < 0 || gate_act >= TNX_ACT_COUNT) return TNX_ERR_BAD_ARG;
    const int warps = 4;
    const long long pairs = (long long)n_tokens * H;
    const int blocks = (int)((pairs + warps - 1) / warps);
    if (is_h16)
        return tnx_launch_in_order(headwise_gated_rms_norm_kernel<h16>, dim3(blocks), dim3(warps * 32), 0, stream, o,
                                   (const h16*)gate, gate_ld, token_request, w, eps, out_scale, (h16*)out, out_ld, n_tokens,
                                   H, dv, gate_act);
    return tnx_launch_in_order(headwise_gated_rms_norm_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o,
                               (const float*)gate, gate_ld, token_request, w, eps, out_scale, (float*)out, out_ld, n_tokens,
                               H, dv, gate_act);
}

// One token per request: rotation, state update, output, head-wise norm, gate and scale in one kernel.  Returns
// TNX_ERR_UNSUPPORTED for sizes it does not take (the caller then runs the three kernels); g_off < 0: no gate.
template <typename T>
static int retention_decode_launch(const T* proj, int ld, int q_off, int k_off, int v_off, int g_off, const int* positions,
                                   const float* inv_freq, int rot_dims, float k_scale, const float* decay, float* state,
                                   const int* q_start, const int* q_len, const int* state_slots, float eps, float out_scale,
                                   T* out, int out_ld, int n_requests, int H, int dk, int dv, cudaStream_t stream) {
    const int CG = (dv + 3) / 4;
#define RDEC(KPT, R)                                                                                                    \
    do {                                                                                                                \
        const int threads = ((CG * (R) + 31) / 32) * 32;                                                                \
        if (threads > 512) return TNX_ERR_UNSUPPORTED;                                                                  \
        const size_t smem = (size_t)(2 * (KPT) * (R) + 3 * 4 * CG + CG * (4 * (R) + 4)) * sizeof(float);                \
        if (smem > 48 * 1024) return TNX_ERR_UNSUPPORTED;                                                               \
        return tnx_launch_in_order(retention_decode_kernel<T, KPT, R>, dim3(H, n_requests), dim3(threads), smem, stream, \
                                   proj, ld, q_off, k_off, v_off, g_off, positions, inv_freq, rot_dims, k_scale, decay, \
                                   state, q_start, q_len, state_slots, eps, out_scale, out, out_ld, H, dk, dv);         \
    } while (0)
    if (dk <= 16) RDEC(4, 4);
    if (dk <= 32) RDEC(4, 8);
    if (dk <= 64) RDEC(4, 16);
    if (dk <= 128) RDEC(8, 16);
    if (dk <= 256) RDEC(16, 16);
    return TNX_ERR_UNSUPPORTED;
#undef RDEC
}

TNX_EXPORT int tnx_retention_decode(const void* proj, int ld, int q_off, int k_off, int v_off, int g_off,
                                    const int* positions, const float* inv_freq, int rot_dims, float k_scale,
                                    const float* decay, float* state, const int* q_start, const int* q_len,
                                    const int* state_slots, float eps, float out_scale, void* out, int out_ld,
                                    int n_requests, int H, int dk, int dv, int is_h16, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || n_requests > 65535 || rot_dims < 0 || rot_dims > dk || rot_dims % 2 ||
        (rot_dims && !inv_freq) || out_ld < H * dv)
        return TNX_ERR_BAD_ARG;
    if (dk % 4 || dv % 4 || ((uintptr_t)state % 16)) return TNX_ERR_UNSUPPORTED;
    if (is_h16)
        return retention_decode_launch<h16>((const h16*)proj, ld, q_off, k_off, v_off, g_off, positions, inv_freq, rot_dims,
                                            k_scale, decay, state, q_start, q_len, state_slots, eps, out_scale, (h16*)out,
                                            out_ld, n_requests, H, dk, dv, stream);
    return retention_decode_launch<float>((const float*)proj, ld, q_off, k_off, v_off, g_off, positions, inv_freq, rot_dims,
                                          k_scale, decay, state, q_start, q_len, state_slots, eps, out_scale, (float*)out,
                                          out_ld, n_requests, H, dk, dv, stream);
}
