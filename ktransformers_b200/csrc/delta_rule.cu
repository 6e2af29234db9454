// The gated delta rule: a recurrent mixer whose matrix state per head is decayed, corrected toward the token's value under the
// token's key, and read under the token's query (libktb200_seq.so).
//
//   ktb200_delta_prep   per token: a causal filter of `taps` taps along time on every channel of the [q | k | v] columns of proj, SiLU, q and k to
//                       unit vectors per head (q also times dim^-1/2), step eta = sigmoid(.), decay a = exp(-rate softplus(. + dt_bias)), rate = exp(A_log);
//                       the last taps - 1 convolution inputs of every sequence portion go to its state row
//   ktb200_delta_scan   per sequence portion and head, tokens in order:
//                           M <- a M ;  r = eta (v - M^T k) ;  M <- M + k r^T ;  y = M^T q
//
// State row of a sequence and layer (fp32): [ S heads x dim x vdim | conv inputs (taps - 1) x channels, oldest first ], read from
// the row seqs[2][s] (or zeros when -1) and written to the row seqs[3][s]: the caller double-buffers the rows.  Storage type T
// (bf16 or float) for proj and the convolution weights; everything from the convolution's sum on is fp32.  The arithmetic of a
// token does not depend on where a portion starts or ends.
#include <cuda_bf16.h>

#include "common.cuh"
#include "seq_common.cuh"

namespace ktb {

__device__ __forceinline__ float dr_sigmoid(float x) { return __fdiv_rn(1.0f, 1.0f + expf(-x)); }
__device__ __forceinline__ float dr_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------------------------------------ convolution, activations, unit vectors, gates
// grid (tokens, blocks of kPrepUnits units); a unit is one head's run of channels: 2 G query / key heads of d channels, then H value
// heads of dv channels, in the order of the columns qkv_off .. of proj: [q G*d | k G*d | v H*dv].  A warp per unit, a lane keeps up to
// kPrepPerLane channels in registers.  The CTAs of a portion's last token also move the last taps - 1 inputs into the state row; the
// first block of every token computes the step sizes and decays.
constexpr int kPrepUnits = 8;
constexpr int kPrepPerLane = 8;      // head size <= 256
template <typename T>
__global__ void __launch_bounds__(kPrepUnits * 32) delta_prep_kernel(const T* __restrict__ proj, long proj_stride, int qkv_off, int b_off, int a_off, const T* __restrict__ conv_w,
                                                                     int taps, const float* __restrict__ a_log, const float* __restrict__ dt_bias, int H, int G, int d, int dv,
                                                                     float unit_eps, const int* __restrict__ seq_of, const int* __restrict__ seqs, int seqs_stride,
                                                                     float* __restrict__ state, long state_stride, long conv_off, float* __restrict__ qn, float* __restrict__ kn,
                                                                     float* __restrict__ vv, float* __restrict__ beta, float* __restrict__ decay) {
    const long t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = seq_of[t];
    const int start = seqs[s], len = seqs[seqs_stride + s], rd = seqs[2 * seqs_stride + s], wr = seqs[3 * seqs_stride + s];
    const int off = (int)t - start, C = 2 * G * d + H * dv, back = taps - 1;
    if (blockIdx.y == 0) {
        for (int h = tid; h < H; h += blockDim.x) {
            beta[t * H + h] = dr_sigmoid(to_f(proj[t * proj_stride + b_off + h]));
            decay[t * H + h] = expf(-expf(a_log[h]) * dr_softplus(to_f(proj[t * proj_stride + a_off + h]) + dt_bias[h]));
        }
    }
    const int unit = blockIdx.y * kPrepUnits + warp;
    if (unit >= 2 * G + H) return;
    const bool is_v = unit >= 2 * G;
    const int n = is_v ? dv : d, c0 = is_v ? 2 * G * d + (unit - 2 * G) * dv : unit * d;
    // input of channel c at the portion's offset i (negative: before this portion, from the state row or zero)
    auto input = [&](int i, int c) -> float {
        if (i >= 0) return to_f(proj[(long)(start + i) * proj_stride + qkv_off + c]);
        return rd >= 0 ? state[(long)rd * state_stride + conv_off + (long)(back + i) * C + c] : 0.f;
    };
    float y[kPrepPerLane];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < kPrepPerLane; e++) {
        const int c = c0 + lane + 32 * e;
        y[e] = 0.f;
        if (lane + 32 * e < n) {
            float a = 0.f;
            for (int j = 0; j < taps; j++) a = fmaf(to_f(conv_w[(long)c * taps + j]), input(off - back + j, c), a);
            y[e] = act_silu(a);
            ss += y[e] * y[e];
        }
    }
    if (off == len - 1 && wr >= 0) {
        for (int j = 0; j < back; j++)
            for (int i = lane; i < n; i += 32) state[(long)wr * state_stride + conv_off + (long)j * C + c0 + i] = input(len - back + j, c0 + i);
    }
    float mul = 1.f;
    if (!is_v) {
        ss = warp_sum(ss);
        mul = 1.0f / sqrtf(ss + unit_eps) * (unit < G ? 1.0f / sqrtf((float)d) : 1.0f);
    }
    float* dst = is_v ? vv + t * (long)(H * dv) + (unit - 2 * G) * dv : (unit < G ? qn + (t * G + unit) * d : kn + (t * G + unit - G) * d);
#pragma unroll
    for (int e = 0; e < kPrepPerLane; e++)
        if (lane + 32 * e < n) dst[lane + 32 * e] = y[e] * mul;
}

// ------------------------------------------------------------------------------------------------ the recurrence
// grid (sequence portions, heads, column blocks of 32 value columns); 8 warps; thread (warp w, lane) keeps S[i][col] for a contiguous
// run of key channels i in registers.  Tokens run in order in chunks of kDeltaChunk staged in shared memory.  With S the state
// before the token (M in the notation above),  M^T k  and  M^T q  are summed over the warps in one pass (one barrier per token); then
//     r = eta (v - a M^T k) ,   M <- a M + k r^T ,   y = a M^T q + (k . q) r       (= M_new^T q)
constexpr int kDeltaChunk = 16;
constexpr int kDeltaWarps = 8;
constexpr int kDeltaRows = 32;         // key channels per thread: dim <= 256
template <int ROWS>
__global__ void __launch_bounds__(256) delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv, const float* __restrict__ beta,
                                                         const float* __restrict__ decay, int H, int G, int d, int dv, const int* __restrict__ seqs, int seqs_stride,
                                                         float* __restrict__ state, long state_stride, float* __restrict__ o_out) {
    extern __shared__ __align__(16) float sm[];
    // warp w owns the key channels w * rpt .. w * rpt + rpt - 1 (rpt a multiple of 4: float4 reads); channels >= d are zero
    const int rpt = (((d + kDeltaWarps - 1) / kDeltaWarps) + 3) & ~3, dp = rpt * kDeltaWarps;
    float* qs = sm;                                   // [chunk][dp]
    float* ks = qs + kDeltaChunk * dp;                // [chunk][dp]
    float* vs = ks + kDeltaChunk * dp;                // [chunk][32]
    float* sc = vs + kDeltaChunk * 32;                // [chunk][4]: decay, beta, k . q
    float2* part = reinterpret_cast<float2*>(sc + kDeltaChunk * 4);      // [chunk][warps][32]
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32, hk = h / (H / G);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, col = c0 + lane;
    const int start = seqs[s], len = seqs[seqs_stride + s], rd = seqs[2 * seqs_stride + s], wr = seqs[3 * seqs_stride + s];
    float S[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; r++) {
        const int i = warp * rpt + r;
        S[r] = (rd >= 0 && r < rpt && i < d && col < dv) ? state[(long)rd * state_stride + ((long)h * d + i) * dv + col] : 0.f;
    }
    for (int t0 = 0; t0 < len; t0 += kDeltaChunk) {
        const int nt = min(kDeltaChunk, len - t0);
        __syncthreads();      // the previous chunk is consumed
        for (int i = threadIdx.x; i < nt * dp; i += blockDim.x) {
            const int tt = i / dp, c = i - tt * dp;
            const long row = (long)(start + t0 + tt);
            qs[i] = c < d ? qn[(row * G + hk) * d + c] : 0.f;
            ks[i] = c < d ? kn[(row * G + hk) * d + c] : 0.f;
        }
        for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
            const int c = c0 + (i & 31);
            vs[i] = c < dv ? vv[((long)(start + t0 + (i >> 5)) * H + h) * dv + c] : 0.f;
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += kDeltaWarps) {
            float a = 0.f;
            for (int i = lane; i < dp; i += 32) a = fmaf(ks[tt * dp + i], qs[tt * dp + i], a);
            a = warp_sum(a);
            if (lane == 0) {
                const long row = (long)(start + t0 + tt);
                sc[tt * 4] = decay[row * H + h];
                sc[tt * 4 + 1] = beta[row * H + h];
                sc[tt * 4 + 2] = a;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float4* qr = reinterpret_cast<const float4*>(qs + tt * dp + warp * rpt);
            const float4* kr = reinterpret_cast<const float4*>(ks + tt * dp + warp * rpt);
            float pk = 0.f, pq = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < ROWS / 4; r4++) {
                if (4 * r4 < rpt) {
                    const float4 k = kr[r4], qv = qr[r4];
                    pk = fmaf(S[4 * r4], k.x, pk);     pq = fmaf(S[4 * r4], qv.x, pq);
                    pk = fmaf(S[4 * r4 + 1], k.y, pk); pq = fmaf(S[4 * r4 + 1], qv.y, pq);
                    pk = fmaf(S[4 * r4 + 2], k.z, pk); pq = fmaf(S[4 * r4 + 2], qv.z, pq);
                    pk = fmaf(S[4 * r4 + 3], k.w, pk); pq = fmaf(S[4 * r4 + 3], qv.w, pq);
                }
            }
            part[(tt * kDeltaWarps + warp) * 32 + lane] = make_float2(pk, pq);
            __syncthreads();
            float sk = 0.f, sq = 0.f;
#pragma unroll
            for (int w = 0; w < kDeltaWarps; w++) {      // every warp sums in the same order: all threads of a column agree on u
                const float2 v = part[(tt * kDeltaWarps + w) * 32 + lane];
                sk += v.x;
                sq += v.y;
            }
            const float g = sc[tt * 4], b = sc[tt * 4 + 1], kq = sc[tt * 4 + 2];
            const float u = b * (vs[tt * 32 + lane] - g * sk);
#pragma unroll
            for (int r4 = 0; r4 < ROWS / 4; r4++) {
                if (4 * r4 < rpt) {
                    const float4 k = kr[r4];
                    S[4 * r4] = fmaf(g, S[4 * r4], k.x * u);
                    S[4 * r4 + 1] = fmaf(g, S[4 * r4 + 1], k.y * u);
                    S[4 * r4 + 2] = fmaf(g, S[4 * r4 + 2], k.z * u);
                    S[4 * r4 + 3] = fmaf(g, S[4 * r4 + 3], k.w * u);
                }
            }
            if (warp == 0 && col < dv) o_out[((long)(start + t0 + tt) * H + h) * dv + col] = fmaf(g, sq, kq * u);
        }
    }
    if (wr >= 0) {
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            const int i = warp * rpt + r;
            if (r < rpt && i < d && col < dv) state[(long)wr * state_stride + ((long)h * d + i) * dv + col] = S[r];
        }
    }
}

}  // namespace ktb

using namespace ktb;

#define GRANT_SMEM(kernel, smem)                                                                                                       \
    do {                                                                                                                               \
        static size_t granted = 48 * 1024;                                                                                             \
        if ((smem) > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem))); granted = (smem); } \
    } while (0)

extern "C" int ktb200_delta_prep(const void* proj, long proj_stride, int qkv_off, int b_off, int a_off, const void* conv_w, int taps, const float* a_log, const float* dt_bias,
                                 int heads, int kv_heads, int dim, int vdim, float unit_eps, const int* seq_of, const int* seqs, int seqs_stride, float* state, long state_stride,
                                 float* qn, float* kn, float* vv, float* beta, float* decay, int n_tokens, int dtype, void* stream) {
    if (!proj || !conv_w || !a_log || !dt_bias || !seq_of || !seqs || !state || !qn || !kn || !vv || !beta || !decay || heads <= 0 || kv_heads <= 0 || heads % kv_heads ||
        dim <= 0 || dim > 32 * kPrepPerLane || vdim <= 0 || vdim > 32 * kPrepPerLane || taps < 1) {
        set_error("delta_prep: bad argument (head sizes <= %d)", 32 * kPrepPerLane);
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    const long conv_off = (long)heads * dim * vdim;
    const dim3 grid(n_tokens, (2 * kv_heads + heads + kPrepUnits - 1) / kPrepUnits);
    if (dtype == KTB200_TYPE_BF16) {
        using T = __nv_bfloat16;
        delta_prep_kernel<T><<<grid, kPrepUnits * 32, 0, (cudaStream_t)stream>>>((const T*)proj, proj_stride, qkv_off, b_off, a_off, (const T*)conv_w, taps, a_log, dt_bias, heads, kv_heads,
                                                                            dim, vdim, unit_eps, seq_of, seqs, seqs_stride, state, state_stride, conv_off, qn, kn, vv, beta, decay);
    } else if (dtype == KTB200_TYPE_F32) {
        using T = float;
        delta_prep_kernel<T><<<grid, kPrepUnits * 32, 0, (cudaStream_t)stream>>>((const T*)proj, proj_stride, qkv_off, b_off, a_off, (const T*)conv_w, taps, a_log, dt_bias, heads, kv_heads,
                                                                            dim, vdim, unit_eps, seq_of, seqs, seqs_stride, state, state_stride, conv_off, qn, kn, vv, beta, decay);
    } else {
        set_error("delta_prep: dtype must be bf16 or f32");
        return KTB200_EINVAL;
    }
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_delta_scan(const float* qn, const float* kn, const float* vv, const float* beta, const float* decay, int heads, int kv_heads, int dim, int vdim,
                                 const int* seqs, int seqs_stride, int n_seqs, float* state, long state_stride, float* o_out, void* stream) {
    if (!qn || !kn || !vv || !beta || !decay || !seqs || !state || !o_out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim > kDeltaWarps * kDeltaRows ||
        vdim <= 0) {
        set_error("delta_scan: bad argument (dim <= %d)", kDeltaWarps * kDeltaRows);
        return KTB200_EINVAL;
    }
    if (n_seqs <= 0) return KTB200_OK;
    const int rpt = (((dim + kDeltaWarps - 1) / kDeltaWarps) + 3) & ~3, dp = rpt * kDeltaWarps;
    const size_t smem = ((size_t)2 * kDeltaChunk * dp + kDeltaChunk * 32 + kDeltaChunk * 4 + (size_t)2 * kDeltaChunk * kDeltaWarps * 32) * sizeof(float);
    const dim3 grid(n_seqs, heads, (vdim + 31) / 32);
#define DELTA_LAUNCH(ROWS)                                                                                                                                       \
    do {                                                                                                                                                         \
        GRANT_SMEM(delta_scan_kernel<ROWS>, smem);                                                                                                               \
        delta_scan_kernel<ROWS><<<grid, kDeltaWarps * 32, smem, (cudaStream_t)stream>>>(qn, kn, vv, beta, decay, heads, kv_heads, dim, vdim, seqs, seqs_stride, state, \
                                                                                        state_stride, o_out);                                                    \
    } while (0)
    if (rpt <= 8) DELTA_LAUNCH(8);
    else if (rpt <= 16) DELTA_LAUNCH(16);
    else DELTA_LAUNCH(32);
#undef DELTA_LAUNCH
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}
