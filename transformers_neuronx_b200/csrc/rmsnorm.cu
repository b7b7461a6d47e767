// RMS norm over the hidden axis, in 32-bit from the 32-bit residual stream, optionally of a sum:
//   y = x_scale * x + delta          (delta: what a sublayer produced; absent: y = x_scale * x)
//   out = y / sqrt(mean(y^2) + eps) * (w + w_offset) * out_scale        (w absent: no weight)
// One thread block per row; the row is kept in shared memory between the two passes, so out_f32
// may be x itself (a post-norm block normalises its residual stream in place).
// `rows`, when given, picks the input rows (the rows whose logits are wanted).
#include "common.cuh"

template <typename TA, bool VEC>
__global__ void rms_norm_kernel(const float* __restrict__ x, float x_scale, const float* __restrict__ delta,
                                const int* __restrict__ rows, const float* __restrict__ w, float w_offset, float eps,
                                float out_scale, float* out_f32, TA* __restrict__ out_act, int H) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    float s = 0.f;
    if (VEC) {
        const float4* xs = (const float4*)(x + src);
        const float4* ds = delta ? (const float4*)(delta + src) : nullptr;
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            float4 v = xs[c];
            v.x *= x_scale; v.y *= x_scale; v.z *= x_scale; v.w *= x_scale;
            if (ds) { const float4 d = ds[c]; v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w; }
            ((float4*)row)[c] = v;
            s += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = x[src + c] * x_scale;
            if (delta) v += delta[src + c];
            row[c] = v;
            s += v * v;
        }
    }
    const float ms = block_sum(s, scratch) / (float)H;
    const float rinv = 1.0f / sqrtf(ms + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float y = row[c] * rinv;
        if (w) y *= (w[c] + w_offset);
        y *= out_scale;
        if (out_f32) out_f32[(size_t)r * H + c] = y;
        if (out_act) out_act[(size_t)r * H + c] = from_float<TA>(y);
    }
}

// Two norms of the same row (the inputs of two sublayers that run side by side on one stream): the mean square is
// formed once,  out1 = x / sqrt(ms + eps1) * (w1 + off1),  out2 = x / sqrt(ms + eps2) * (w2 + off2).
template <typename TA>
__global__ void rms_norm_pair_kernel(const float* __restrict__ x, const float* __restrict__ w1, float off1, float eps1,
                                     const float* __restrict__ w2, float off2, float eps2, TA* __restrict__ out1,
                                     TA* __restrict__ out2, int H) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t src = (size_t)blockIdx.x * H;
    float s = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = x[src + c];
        row[c] = v;
        s += v * v;
    }
    const float ms = block_sum(s, scratch) / (float)H;
    const float r1 = 1.0f / sqrtf(ms + eps1), r2 = 1.0f / sqrtf(ms + eps2);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = row[c];
        out1[src + c] = from_float<TA>(v * r1 * (w1 ? w1[c] + off1 : 1.f));
        if (out2) out2[src + c] = from_float<TA>(v * r2 * (w2 ? w2[c] + off2 : 1.f));
    }
}

// x <- x + s1 * a (+ s2 * b): two sublayers' results, each multiplied channel by channel by a learned scale, enter
// the 32-bit stream in one pass (s1, s2 absent: 1; b absent: one sublayer).  With out1 the new row's norms for the two
// sublayers of the layer that follows are formed in the same kernel (the row stays in shared memory):
// out_i = x / sqrt(mean(x^2) + eps_i) * (w_i + off_i), out2 optional.
template <typename TA>
__global__ void scaled_residual_add_kernel(float* x, const float* __restrict__ a, const float* __restrict__ s1,
                                           const float* __restrict__ b, const float* __restrict__ s2, int H,
                                           const float* __restrict__ w1, float off1, float eps1, TA* __restrict__ out1,
                                           const float* __restrict__ w2, float off2, float eps2, TA* __restrict__ out2) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t src = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float d = a[src + c] * (s1 ? s1[c] : 1.f);
        if (b) d = fmaf(b[src + c], s2 ? s2[c] : 1.f, d);
        const float v = x[src + c] + d;
        x[src + c] = v;
        if (out1) { row[c] = v; ss = fmaf(v, v, ss); }
    }
    if (!out1) return;
    const float ms = block_sum(ss, scratch) / (float)H;
    const float r1 = 1.0f / sqrtf(ms + eps1), r2 = 1.0f / sqrtf(ms + eps2);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {           // a thread reads back what it wrote itself
        const float v = row[c];
        out1[src + c] = from_float<TA>(v * r1 * (w1 ? w1[c] + off1 : 1.f));
        if (out2) out2[src + c] = from_float<TA>(v * r2 * (w2 ? w2[c] + off2 : 1.f));
    }
}

// Four neighbouring elements stored at once (8 bytes of 16-bit numbers, 16 of floats).
__device__ __forceinline__ void store4(float* p, const float4& v) { *(float4*)p = v; }
__device__ __forceinline__ void store4(h16* p, const float4& v) {
    uint2 raw;
    *(h16x2*)&raw.x = floats_to_h16x2(v.x, v.y);
    *(h16x2*)&raw.y = floats_to_h16x2(v.z, v.w);
    *(uint2*)p = raw;
}

// The norm on a sublayer's output only:  out = x + add_scale * (delta / sqrt(mean(delta^2) + eps) * (w + w_offset)).
// x is the 32-bit residual stream (out_f32 may be x itself), delta what the sublayer produced.
// then_norm: out_act receives a further RMS norm of the new row, out / sqrt(mean(out^2) + then_eps) * (w_then + then_offset),
// which is the input of the sublayer that follows (a norm before and after every sublayer); otherwise the row's copy.
template <typename TA, bool VEC>
__global__ void rms_norm_add_kernel(const float* x, float add_scale, const float* __restrict__ delta,
                                    const float* __restrict__ w, float w_offset, float eps, float* out_f32,
                                    TA* __restrict__ out_act, int H, int then_norm, const float* __restrict__ w_then,
                                    float then_offset, float then_eps) {
    extern __shared__ __align__(16) float row[];      // the sublayer's row; with VEC the stream's row behind it
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t src = (size_t)blockIdx.x * H;
    float s = 0.f;
    if (VEC) {
        // sixteen bytes an access throughout, and the stream's row fetched along with the sublayer's, so that nothing
        // is waited for behind the first sum
        const float4* ds = (const float4*)(delta + src);
        const float4* xs = (const float4*)(x + src);
        float4* rd = (float4*)row;
        float4* rx = (float4*)(row + H);
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            const float4 v = ds[c];
            rd[c] = v;
            rx[c] = xs[c];
            s += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        const float rinv = 1.0f / sqrtf(block_sum(s, scratch) / (float)H + eps);
        float s2 = 0.f;
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            float4 y = rd[c];
            const float4 xv = rx[c];
            y.x *= rinv; y.y *= rinv; y.z *= rinv; y.w *= rinv;
            if (w) {
                const float4 g = ((const float4*)w)[c];
                y.x *= g.x + w_offset; y.y *= g.y + w_offset; y.z *= g.z + w_offset; y.w *= g.w + w_offset;
            }
            y.x = fmaf(add_scale, y.x, xv.x); y.y = fmaf(add_scale, y.y, xv.y);
            y.z = fmaf(add_scale, y.z, xv.z); y.w = fmaf(add_scale, y.w, xv.w);
            if (out_f32) ((float4*)(out_f32 + src))[c] = y;
            if (then_norm) { rd[c] = y; s2 += (y.x * y.x + y.y * y.y) + (y.z * y.z + y.w * y.w); }
            else if (out_act) store4(out_act + src + 4 * c, y);
        }
        if (!then_norm || !out_act) return;
        const float rinv2 = 1.0f / sqrtf(block_sum(s2, scratch) / (float)H + then_eps);  // each thread reads back its own columns
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            float4 y = rd[c];
            y.x *= rinv2; y.y *= rinv2; y.z *= rinv2; y.w *= rinv2;
            if (w_then) {
                const float4 g = ((const float4*)w_then)[c];
                y.x *= g.x + then_offset; y.y *= g.y + then_offset; y.z *= g.z + then_offset; y.w *= g.w + then_offset;
            }
            store4(out_act + src + 4 * c, y);
        }
        return;
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = delta[src + c];
        row[c] = v;
        s += v * v;
    }
    const float ms = block_sum(s, scratch) / (float)H;
    const float rinv = 1.0f / sqrtf(ms + eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float y = row[c] * rinv;
        if (w) y *= (w[c] + w_offset);
        y = fmaf(add_scale, y, x[src + c]);
        if (out_f32) out_f32[src + c] = y;
        if (then_norm) { row[c] = y; s2 += y * y; }
        else if (out_act) out_act[src + c] = from_float<TA>(y);
    }
    if (!then_norm || !out_act) return;
    const float rinv2 = 1.0f / sqrtf(block_sum(s2, scratch) / (float)H + then_eps);     // each thread reads back its own columns
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float y = row[c] * rinv2;
        if (w_then) y *= (w_then[c] + then_offset);
        out_act[src + c] = from_float<TA>(y);
    }
}

TNX_EXPORT int tnx_rms_norm_add(const float* x, float add_scale, const float* delta, const float* w, float w_offset,
                                float eps, float* out_f32, void* out_act, int n_rows, int H, int act_h16,
                                int then_norm, const float* w_then, float then_offset, float then_eps,
                                cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || !x || !delta) return TNX_ERR_UNSUPPORTED;
    const bool vec = H % 4 == 0 && (size_t)2 * H * sizeof(float) <= 200 * 1024 &&
                     !(((uintptr_t)delta | (uintptr_t)x | (uintptr_t)out_f32 | (uintptr_t)out_act | (uintptr_t)w |
                        (uintptr_t)w_then) & 15);
    const size_t smem = (size_t)(vec ? 2 : 1) * H * sizeof(float);
    if (smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
#define RMS_LAUNCH(TA, V)                                                                                              \
    do {                                                                                                               \
        if (smem + 1024 > 48 * 1024)                                                                                   \
            cudaFuncSetAttribute(rms_norm_add_kernel<TA, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        return tnx_launch_ex(1, rms_norm_add_kernel<TA, V>, dim3(n_rows), dim3(threads), smem, stream, x, add_scale,   \
                             delta, w, w_offset, eps, out_f32, (TA*)out_act, H, then_norm, w_then, then_offset,        \
                             then_eps);                                                                                \
    } while (0)
    if (act_h16) { if (vec) RMS_LAUNCH(h16, true); else RMS_LAUNCH(h16, false); }
    if (vec) RMS_LAUNCH(float, true); else RMS_LAUNCH(float, false);
#undef RMS_LAUNCH
}

TNX_EXPORT int tnx_rms_norm_pair(const float* x, const float* w1, float off1, float eps1, const float* w2, float off2,
                                 float eps2, void* out1, void* out2, int n_rows, int H, int act_h16, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    if (H <= 0 || !x || !out1 || smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (act_h16) {
        if (smem + 1024 > 48 * 1024)
            cudaFuncSetAttribute(rms_norm_pair_kernel<h16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tnx_launch_ex(1, rms_norm_pair_kernel<h16>, dim3(n_rows), dim3(threads), smem, stream, x, w1, off1, eps1, w2,
                             off2, eps2, (h16*)out1, (h16*)out2, H);
    }
    if (smem + 1024 > 48 * 1024)
        cudaFuncSetAttribute(rms_norm_pair_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return tnx_launch_ex(1, rms_norm_pair_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, w1, off1, eps1, w2,
                         off2, eps2, (float*)out1, (float*)out2, H);
}

TNX_EXPORT int tnx_scaled_residual_add(float* x, const float* a, const float* s1, const float* b, const float* s2,
                                       int n_rows, int H, const float* w1, float off1, float eps1, void* out1,
                                       const float* w2, float off2, float eps2, void* out2, int act_h16,
                                       cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || !x || !a || (out2 && !out1)) return TNX_ERR_BAD_ARG;
    const size_t smem = out1 ? (size_t)H * sizeof(float) : 0;
    if (smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (act_h16) {
        if (smem + 1024 > 48 * 1024)
            cudaFuncSetAttribute(scaled_residual_add_kernel<h16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tnx_launch_ex(1, scaled_residual_add_kernel<h16>, dim3(n_rows), dim3(threads), smem, stream, x, a, s1, b, s2, H,
                             w1, off1, eps1, (h16*)out1, w2, off2, eps2, (h16*)out2);
    }
    if (smem + 1024 > 48 * 1024)
        cudaFuncSetAttribute(scaled_residual_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return tnx_launch_ex(1, scaled_residual_add_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, a, s1, b, s2, H,
                         w1, off1, eps1, (float*)out1, w2, off2, eps2, (float*)out2);
}

TNX_EXPORT int tnx_rms_norm(const float* x, float x_scale, const float* delta, const int* rows, const float* w,
                            float w_offset, float eps, float out_scale, float* out_f32, void* out_act, int n_rows, int H,
                            int act_h16, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    if (H <= 0 || smem > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const bool vec = H % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)delta % 16) == 0;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
#define RMS_LAUNCH(TA, V)                                                                                              \
    do {                                                                                                               \
        if (smem + 1024 > 48 * 1024)                                                                                   \
            cudaFuncSetAttribute(rms_norm_kernel<TA, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        return tnx_launch_ex(1, rms_norm_kernel<TA, V>, dim3(n_rows), dim3(threads), smem, stream, x, x_scale, delta,  \
                             rows, w, w_offset, eps, out_scale, out_f32, (TA*)out_act, H);                             \
    } while (0)
    if (act_h16) { if (vec) RMS_LAUNCH(h16, true); else RMS_LAUNCH(h16, false); }
    if (vec) RMS_LAUNCH(float, true); else RMS_LAUNCH(float, false);
#undef RMS_LAUNCH
}
