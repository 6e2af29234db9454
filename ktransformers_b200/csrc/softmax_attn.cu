// Soft-max attention over grouped key/value heads in a paged cache, with a partial rotation, unit-rms queries and keys, capped
// scores, a sliding window and values blended with another layer's (libktb200_seq.so).
//
//   ktb200_rope_norm_cache_write   proj rows [... q H*d ... k G*d ... v G*dv ...]: q and k turn over their first rot_dims columns (pairs of
//                                  either layout, angle pos * inv_freq[i]), are scaled to unit rms head by head (optional),
//                                  v <- (1 - t) v + t v_other with one learned t (optional); [k | v] into the paged cache, q into q_out
//   ktb200_window_softmax_attn     o_i = sum_j softmax_j(cap(scale q_i.k_j)) v_j over the keys j with 0 <= i - j < window (window <= 0: all
//                                  j <= i), cap(s) = c tanh(s / c), c = softcap (softcap <= 0: none); query head h reads key/value
//                                  head h / (H / G); the key range is cut into splits for few tokens on long ranges
//
// Storage type T (bf16 or float) for activations and cache rows; rotation, norms, scores, the cap and the soft-max are fp32
// (angles fp64).  Cache row of a token: [k G*d | v G*dv]; a sequence's page table row is a ring.
#include <cuda_bf16.h>

#include "common.cuh"
#include "seq_common.cuh"

namespace ktb {

// ------------------------------------------------------------------------------------------------ rotation, unit rms, value blend, cache write
// One CTA per token, a warp per head (query heads first, then key heads).
constexpr int kPrepMaxPerLane = 8;      // head size <= 256
template <typename T>
__global__ void __launch_bounds__(256) rope_norm_cache_write_kernel(const T* __restrict__ proj, long proj_stride, int q_off, int k_off, int v_off, int H, int G, int d, int dv,
                                                                    int rot_dims, int rot_layout, const double* __restrict__ inv_freq, int unit_rms, float eps,
                                                                    const T* __restrict__ v_other, long v_other_stride, const float* __restrict__ blend,
                                                                    const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ page_table,
                                                                    int max_pages, int page_size, T* __restrict__ cache, T* __restrict__ q_out) {
    const long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int p = pos[t];
    const T* row = proj + t * proj_stride;
    const long crow = ((long)page_table[(long)slot[t] * max_pages + (p / page_size) % max_pages] * page_size + p % page_size) * ((long)G * (d + dv));
    for (int hh = warp; hh < H + G; hh += nw) {
        const bool is_q = hh < H;
        const T* src = is_q ? row + q_off + (long)hh * d : row + k_off + (long)(hh - H) * d;
        float r[kPrepMaxPerLane];
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < kPrepMaxPerLane; e++) {
            const int i = lane + 32 * e;
            r[e] = 0.f;
            if (i < d) {
                float v = to_f(src[i]);
                if (i < rot_dims) v = rot_turn(v, to_f(src[rot_partner(i, rot_dims, rot_layout)]), i, rot_dims, rot_layout, p, inv_freq);
                r[e] = v;
                s += v * v;
            }
        }
        float inv = 1.f;
        if (unit_rms) {
            s = warp_sum(s);
            inv = 1.0f / sqrtf(s / (float)d + eps);
        }
        T* dst = is_q ? q_out + (t * H + hh) * d : cache + crow + (long)(hh - H) * d;
#pragma unroll
        for (int e = 0; e < kPrepMaxPerLane; e++) {
            const int i = lane + 32 * e;
            if (i < d) dst[i] = from_f<T>(r[e] * inv);
        }
    }
    const T* v = row + v_off;
    const float lam = v_other ? blend[0] : 0.f;
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x) {
        float x = to_f(v[i]);
        if (v_other) x = (1.0f - lam) * x + lam * to_f(v_other[t * v_other_stride + i]);
        cache[crow + (long)G * d + i] = from_f<T>(x);
    }
}

// ------------------------------------------------------------------------------------------------ soft-max attention, CUDA cores
// grid (tokens, G * head blocks, splits); a warp per query head (HB = blockDim / 32 heads of ONE key/value head per CTA).  Tiles of
// 32 keys in shared memory as fp32: lane = key for the scores, lane = value column for the weighted sum; running maximum and sum per
// warp.  Shared memory:  q [HB][d] | K [32][d + 1] | V [32][dv] | weights [HB][32]
constexpr int kSmTile = 32;
constexpr int kSmMaxCols = 8;      // value columns per lane: vdim <= 256
__device__ __forceinline__ float cap_score(float s, float softcap) { return softcap > 0.f ? softcap * tanhf(s / softcap) : s; }

template <typename T>
__global__ void __launch_bounds__(256) window_softmax_attn_kernel(const T* __restrict__ q, int H, int G, int d, int dv, float scale, float softcap, int window,
                                                                  const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ page_table,
                                                                  int max_pages, int page_size, const T* __restrict__ cache, T* __restrict__ out,
                                                                  float* __restrict__ partial, int n_tokens) {
    extern __shared__ __align__(16) float sm[];
    const int HB = blockDim.x >> 5, R = H / G, hblocks = (R + HB - 1) / HB;
    const int g = blockIdx.y / hblocks, hb = blockIdx.y % hblocks;
    const long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = hb * HB + warp, h = g * R + r;
    const bool live = r < R;
    float* qs = sm;
    float* Ks = qs + HB * d;
    float* Vs = Ks + kSmTile * (d + 1);
    float* pw = Vs + kSmTile * dv;
    const int p = pos[t];
    // this split's part of the visible range [lo, p], in whole tiles counted from lo
    const int lo = window > 0 ? max(0, p - window + 1) : 0, n_keys = p + 1 - lo;
    const int splits = gridDim.z;
    const int per = ((n_keys + splits - 1) / splits + kSmTile - 1) / kSmTile * kSmTile;
    const int k_lo = lo + blockIdx.z * per, k_hi = min(p + 1, k_lo + per);
    float acc[kSmMaxCols];
#pragma unroll
    for (int c = 0; c < kSmMaxCols; c++) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (k_lo < k_hi) {
        if (live)
            for (int i = lane; i < d; i += 32) qs[warp * d + i] = to_f(q[(t * H + h) * d + i]) * scale;
        const int* pt = page_table + (long)slot[t] * max_pages;
        const long cw = (long)G * (d + dv);
        for (int j0 = k_lo; j0 < k_hi; j0 += kSmTile) {
            __syncthreads();
            const int nk = min(kSmTile, k_hi - j0);
            for (int i = threadIdx.x; i < nk * d; i += blockDim.x) {
                const int j = i / d, c = i - j * d, kp = j0 + j;
                Ks[j * (d + 1) + c] = to_f(cache[((long)pt[(kp / page_size) % max_pages] * page_size + kp % page_size) * cw + (long)g * d + c]);
            }
            for (int i = threadIdx.x; i < nk * dv; i += blockDim.x) {
                const int j = i / dv, c = i - j * dv, kp = j0 + j;
                Vs[j * dv + c] = to_f(cache[((long)pt[(kp / page_size) % max_pages] * page_size + kp % page_size) * cw + (long)G * d + (long)g * dv + c]);
            }
            __syncthreads();
            if (!live) continue;
            float s = -INFINITY;
            if (lane < nk) {
                float a = 0.f;
                const float* kr = Ks + lane * (d + 1);
                const float* qr = qs + warp * d;
                for (int i = 0; i < d; i++) a = fmaf(qr[i], kr[i], a);
                s = cap_score(a, softcap);
            }
            const float mn = fmaxf(m, warp_max(s));      // every tile holds at least one key, so mn is finite
            const float corr = expf(m - mn);
            const float pj = expf(s - mn);
            l = l * corr + warp_sum(pj);
            m = mn;
            pw[warp * kSmTile + lane] = pj;
            __syncwarp();
#pragma unroll
            for (int c = 0; c < kSmMaxCols; c++) acc[c] *= corr;
            for (int j = 0; j < nk; j++) {
                const float wj = pw[warp * kSmTile + j];
#pragma unroll
                for (int c = 0; c < kSmMaxCols; c++)
                    if (lane + 32 * c < dv) acc[c] = fmaf(wj, Vs[j * dv + lane + 32 * c], acc[c]);
            }
            __syncwarp();
        }
    }
    if (!live) return;
    if (partial) {      // [T][H][splits][dv + 2]: running maximum, sum, un-normalised weighted values
        float* o = partial + (((long)t * H + h) * splits + blockIdx.z) * (dv + 2);
        if (lane == 0) { o[0] = m; o[1] = l; }
#pragma unroll
        for (int c = 0; c < kSmMaxCols; c++)
            if (lane + 32 * c < dv) o[2 + lane + 32 * c] = acc[c];
    } else {
        const float inv = 1.0f / l;
#pragma unroll
        for (int c = 0; c < kSmMaxCols; c++)
            if (lane + 32 * c < dv) out[(t * H + h) * dv + lane + 32 * c] = from_f<T>(acc[c] * inv);
    }
}

// one warp per (token, head): the parts' weights exp(m_s - m) / l (parts without a key have m = -inf and weigh nothing), then
// the columns in parallel, parts in order
template <typename T>
__global__ void __launch_bounds__(256) softmax_merge_kernel(const float* __restrict__ partial, int splits, T* __restrict__ out, long n_rows, int dv) {
    const int lane = threadIdx.x & 31;
    for (long row = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows; row += (long)gridDim.x * (blockDim.x >> 5)) {
        const float* part = partial + row * splits * (dv + 2);
        float m = -INFINITY;
        for (int s = lane; s < splits; s += 32) m = fmaxf(m, part[(long)s * (dv + 2)]);
        m = warp_max(m);
        float l = 0.f;
        for (int s = lane; s < splits; s += 32) {
            const float ms = part[(long)s * (dv + 2)];
            if (ms > -INFINITY) l += part[(long)s * (dv + 2) + 1] * expf(ms - m);
        }
        l = warp_sum(l);
        for (int c = lane; c < dv; c += 32) {
            float a = 0.f;
            for (int s = 0; s < splits; s++) {
                const float ms = part[(long)s * (dv + 2)];
                if (ms > -INFINITY) a = fmaf(expf(ms - m), part[(long)s * (dv + 2) + 2 + c], a);
            }
            out[row * dv + c] = from_f<T>(a / l);
        }
    }
}

}  // namespace ktb

using namespace ktb;

#define SEQ_DISPATCH(dtype, ...)                                                           \
    do {                                                                                   \
        if ((dtype) == KTB200_TYPE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }         \
        else if ((dtype) == KTB200_TYPE_F32) { using T = float; __VA_ARGS__; }             \
        else { set_error("dtype must be bf16 or f32"); return KTB200_EINVAL; }             \
    } while (0)
#define GRANT_SMEM(kernel, smem)                                                                                                       \
    do {                                                                                                                               \
        static size_t granted = 48 * 1024;                                                                                             \
        if ((smem) > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem))); granted = (smem); } \
    } while (0)

extern "C" int ktb200_rope_norm_cache_write(const void* proj, long proj_stride, int q_off, int k_off, int v_off, int heads, int kv_heads, int dim, int vdim, int rot_dims,
                                            int rot_layout, const double* inv_freq, int unit_rms, float eps, const void* v_other, long v_other_stride, const float* blend,
                                            const int* pos, const int* slot, const int* page_table, int max_pages, int page_size, void* cache, void* q_out, int n_tokens,
                                            int dtype, void* stream) {
    if (!proj || !pos || !slot || !page_table || !cache || !q_out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim > 32 * kPrepMaxPerLane || vdim <= 0 ||
        rot_dims < 0 || rot_dims > dim || (rot_dims & 1) || (rot_dims && !inv_freq) || (rot_layout != kRotInterleaved && rot_layout != kRotHalves) || (v_other && !blend) ||
        page_size <= 0 || max_pages <= 0) {
        set_error("rope_norm_cache_write: bad argument (head size <= %d)", 32 * kPrepMaxPerLane);
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (rope_norm_cache_write_kernel<T><<<n_tokens, 256, 0, (cudaStream_t)stream>>>(
                            (const T*)proj, proj_stride, q_off, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, rot_layout, inv_freq, unit_rms, eps, (const T*)v_other,
                            v_other_stride, blend, pos, slot, page_table, max_pages, page_size, (T*)cache, (T*)q_out)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" size_t ktb200_window_softmax_attn_workspace(int n_tokens, int heads, int vdim, int splits) {
    return splits > 1 ? (size_t)n_tokens * heads * splits * (vdim + 2) * sizeof(float) : 0;
}

extern "C" int ktb200_window_softmax_attn(const void* q, int heads, int kv_heads, int dim, int vdim, float scale, float softcap, int window, const int* pos, const int* slot,
                                          const int* page_table, int max_pages, int page_size, const void* cache, void* out, int n_tokens, int splits, float* workspace,
                                          int dtype, void* stream) {
    if (!q || !pos || !slot || !page_table || !cache || !out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || vdim > 32 * kSmMaxCols ||
        splits < 1 || (splits > 1 && !workspace) || page_size <= 0 || max_pages <= 0) {
        set_error("window_softmax_attn: bad argument (value size <= %d)", 32 * kSmMaxCols);
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    const int R = heads / kv_heads, HB = R < 8 ? R : 8, hblocks = (R + HB - 1) / HB;
    const size_t smem = ((size_t)HB * dim + (size_t)kSmTile * (dim + 1) + (size_t)kSmTile * vdim + (size_t)HB * kSmTile) * sizeof(float);
    if (smem > 200 * 1024) { set_error("window_softmax_attn: head too wide for shared memory"); return KTB200_EINVAL; }
    SEQ_DISPATCH(dtype, {
        GRANT_SMEM(window_softmax_attn_kernel<T>, smem);
        window_softmax_attn_kernel<T><<<dim3(n_tokens, kv_heads * hblocks, splits), HB * 32, smem, (cudaStream_t)stream>>>(
            (const T*)q, heads, kv_heads, dim, vdim, scale, softcap, window, pos, slot, page_table, max_pages, page_size, (const T*)cache, (T*)out,
            splits > 1 ? workspace : nullptr, n_tokens);
        KTB_LAUNCH_CHECK();
        if (splits > 1) {
            const long rows = (long)n_tokens * heads;
            const long blocks = (rows + 7) / 8;
            softmax_merge_kernel<T><<<(int)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, (cudaStream_t)stream>>>(workspace, splits, (T*)out, rows, vdim);
            KTB_LAUNCH_CHECK();
        }
    });
    return KTB200_OK;
}
