// Storage-type helpers of the token-major operators (seq_ops.cu, window_attn.cu): T is bf16 or float, arithmetic is fp32.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace ktb {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// sum over the CTA; red: >= blockDim.x / 32 floats; every thread gets the same value
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = lane < nw ? red[lane] : 0.f;
    s = warp_sum(s);
    __syncthreads();
    return s;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// four consecutive values (index a multiple of 4, rows 16- / 8-byte aligned) of an fp32 or bf16 array chosen at run time
__device__ __forceinline__ float4 load4_hidden(const void* base, long idx, int type) {
    if (type == KTB200_TYPE_BF16) {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + idx);
        return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
    }
    return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
}
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) { return load4_hidden(p, 0, KTB200_TYPE_BF16); }
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// Partial dot product of a weight row with a vector held in shared memory (fp32), over the columns this lane owns.  Rows whose
// byte length is a multiple of 16 (and 16-byte aligned) stream as 16-byte read-only loads; any other row element by element.
__device__ __forceinline__ float lane_dot(const __nv_bfloat16* __restrict__ w, const float* __restrict__ xs, int n, int lane, bool vec) {
    float s = 0.f;
    if (vec) {
        for (int i = lane * 8; i < n; i += 256) {
            const uint4 v = ldg_stream16(w + i);
            const float4 a = *reinterpret_cast<const float4*>(xs + i), b = *reinterpret_cast<const float4*>(xs + i + 4);
            s = fmaf(__uint_as_float(v.x << 16), a.x, s);
            s = fmaf(__uint_as_float(v.x & 0xffff0000u), a.y, s);
            s = fmaf(__uint_as_float(v.y << 16), a.z, s);
            s = fmaf(__uint_as_float(v.y & 0xffff0000u), a.w, s);
            s = fmaf(__uint_as_float(v.z << 16), b.x, s);
            s = fmaf(__uint_as_float(v.z & 0xffff0000u), b.y, s);
            s = fmaf(__uint_as_float(v.w << 16), b.z, s);
            s = fmaf(__uint_as_float(v.w & 0xffff0000u), b.w, s);
        }
    } else {
        for (int i = lane; i < n; i += 32) s = fmaf(__bfloat162float(w[i]), xs[i], s);
    }
    return s;
}
__device__ __forceinline__ float lane_dot(const float* __restrict__ w, const float* __restrict__ xs, int n, int lane, bool vec) {
    float s = 0.f;
    if (vec) {
        for (int i = lane * 4; i < n; i += 128) {
            const uint4 v = ldg_stream16(w + i);
            const float4 a = *reinterpret_cast<const float4*>(xs + i);
            s = fmaf(__uint_as_float(v.x), a.x, s);
            s = fmaf(__uint_as_float(v.y), a.y, s);
            s = fmaf(__uint_as_float(v.z), a.z, s);
            s = fmaf(__uint_as_float(v.w), a.w, s);
        }
    } else {
        for (int i = lane; i < n; i += 32) s = fmaf(w[i], xs[i], s);
    }
    return s;
}
// Rotary pairs over the first rot_dims columns of a vector.  layout 0: columns (2i, 2i + 1) pair up; layout 1: column i pairs with
// column i + rot_dims / 2.  A pair (x, y) at position pos becomes (x c - y s, y c + x s) with (c, s) = (cos, sin) of pos * inv_freq[i]
// (fp64 table and angle).  `rot_partner`: the column that column c (< rot_dims) turns with; `rot_turn`: the turned value of column c.
constexpr int kRotInterleaved = 0, kRotHalves = 1;
__device__ __forceinline__ int rot_partner(int c, int rot_dims, int layout) {
    const int half = rot_dims >> 1;
    return layout == kRotHalves ? (c < half ? c + half : c - half) : (c ^ 1);
}
__device__ __forceinline__ float rot_turn(float own, float other, int c, int rot_dims, int layout, int pos, const double* __restrict__ inv_freq) {
    const int half = rot_dims >> 1;
    const bool second = layout == kRotHalves ? c >= half : (c & 1);
    const int i = layout == kRotHalves ? (second ? c - half : c) : (c >> 1);
    double sn, cs;
    sincos((double)pos * inv_freq[i], &sn, &cs);
    return second ? own * (float)cs + other * (float)sn : own * (float)cs - other * (float)sn;
}

// Gated feed-forward activations, fp32: what becomes of a (gate, up) pair of pre-activations.
//   kActSilu        silu(g) * u
//   kActGeluTanh    gelu(g) * u, gelu in its tanh form
//   kActClampedGlu  g' = min(g, limit), u' = clamp(u, -limit, limit);  g' sigmoid(1.702 g') (u' + 1)
constexpr int kActSilu = 0, kActGeluTanh = 1, kActClampedGlu = 2;
__device__ __forceinline__ float act_gelu_tanh(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
__device__ __forceinline__ float gated_act(float g, float u, int act, float limit) {
    if (act == kActClampedGlu) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return __fdiv_rn(g, 1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return (act == kActGeluTanh ? act_gelu_tanh(g) : act_silu(g)) * u;
}

template <typename T> __device__ __forceinline__ bool rows_vectorise(const T* base, int n) {
    return (n * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
}

}  // namespace ktb
