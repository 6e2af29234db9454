// Absorbed latent attention over a paged latent cache with a sliding window and a soft-max sink (libktb200_seq.so).
//
// Cache row of a token: [ latent c (R) | rotated key part (dr) ], shared by all heads.  With the key up-projection folded into
// the query (qa_h = W_uk,h^T q_h, done by the caller as a batched product) the score of head h is
//     s = (qa_h . c + rot(q_r,h) . k_r) * scale ,
// the query at position i sees the keys at positions j with 0 <= i - j < window (window <= 0: all j <= i), the soft-max
// denominator holds one extra term exp(sink_h) without a value, and the output is the probability-weighted sum of the latents
// (the value up-projection W_uv,h follows as another batched product).
//
// latent_window_attn_kernel   CTA = (token, group of <= 8 heads); one warp per head; tiles of 32 cached rows are staged in
//                             shared memory once for all heads of the group; lane = key in the score phase, lane = latent
//                             column in the value phase; online soft-max in fp32 starting from (max = sink, sum = 1).
//                             Prompt portions: one CTA per token, the window bounds the work per token.
// latent_window_attn_split    decode-sized batches with long windows: the key range of a (token, head group) is cut into
//                             `splits` parts, each CTA writes (max, sum, un-normalised sum of latents); latent_window_merge
//                             folds the parts and the sink.
// The rotation of the query's rotated part (pairs of either layout, fp64 angle tables) happens in the prologue.
#include <cuda_bf16.h>

#include "common.cuh"
#include "seq_common.cuh"

namespace ktb {

struct WinAttnParams {
    const void* q;        // [T][H][dn + dr]
    const void* q_abs;    // [T][H][R]
    const double* inv_freq;
    const float* sink;    // [H] or null
    const int* pos;
    const int* slot;
    const int* page_table;
    const void* cache;    // [pages][page_size][R + dr]
    void* out;            // [T][H][R]
    float* part;          // split path: [T][H][splits][R + 2]
    int T, H, dn, dr, R, rot_dims, rot_layout, window, max_pages, page_size, row_pad, splits;
    float scale;
};

constexpr int kWinWarps = 8, kWinTile = 32;

template <typename T, int NI, bool SPLIT>
__global__ void __launch_bounds__(kWinWarps * 32) latent_window_attn_kernel(const WinAttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = p.R, dr = p.dr, RS = R + dr, RSP = RS + p.row_pad;
    float* qa = reinterpret_cast<float*>(smem_raw);                 // [warps][R]
    float* qr = qa + kWinWarps * R;                                  // [warps][dr]
    float* pw = qr + kWinWarps * dr;                                 // [warps][32]
    T* tile = reinterpret_cast<T*>(pw + kWinWarps * kWinTile);       // [32][RSP]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * kWinWarps + warp;
    const bool live = h < p.H;
    const int pos = p.pos[t];
    const T* cache = reinterpret_cast<const T*>(p.cache);
    const int* pt = p.page_table + (long)p.slot[t] * p.max_pages;
    int j0 = p.window > 0 ? max(0, pos - p.window + 1) : 0, j1 = pos + 1;
    if (SPLIT) {   // this CTA's part of [j0, j1), in whole tiles
        const int ntile = (j1 - j0 + kWinTile - 1) / kWinTile, per = (ntile + p.splits - 1) / p.splits;
        const int a = j0 + (int)blockIdx.z * per * kWinTile;
        j1 = min(j1, a + per * kWinTile);
        j0 = a;
    }
    if (live) {
        const T* q = reinterpret_cast<const T*>(p.q) + ((long)t * p.H + h) * (p.dn + dr) + p.dn;
        for (int i = lane; i < dr; i += 32) {
            float v = to_f(q[i]);
            if (i < p.rot_dims) v = rot_turn(v, to_f(q[rot_partner(i, p.rot_dims, p.rot_layout)]), i, p.rot_dims, p.rot_layout, pos, p.inv_freq);
            qr[warp * dr + i] = v;
        }
        const T* a = reinterpret_cast<const T*>(p.q_abs) + ((long)t * p.H + h) * R;
        for (int i = lane; i < R; i += 32) qa[warp * R + i] = to_f(a[i]);
    }
    float m = (!SPLIT && p.sink && live) ? p.sink[h] : -INFINITY;
    float l = (!SPLIT && p.sink && live) ? 1.0f : 0.0f;
    constexpr int VW = sizeof(T) == 2 ? 2 : 1;      // bf16: a lane owns column PAIRS (32-bit shared-memory loads in the value phase)
    auto col = [&](int i) { return VW == 2 ? 2 * (lane + 32 * (i >> 1)) + (i & 1) : lane + 32 * i; };
    float acc[NI];
#pragma unroll
    for (int i = 0; i < NI; i++) acc[i] = 0.f;

    const bool words = (RS * sizeof(T)) % 4 == 0 && (RSP * sizeof(T)) % 4 == 0;
    for (int jt = j0; jt < j1; jt += kWinTile) {
        __syncthreads();   // the previous tile is consumed (and qa / qr are written, first time round)
        for (int r = warp; r < kWinTile; r += kWinWarps) {
            const int j = jt + r;
            T* dst = tile + (long)r * RSP;
            if (j < j1) {
                const T* src = cache + ((long)pt[(j / p.page_size) % p.max_pages] * p.page_size + j % p.page_size) * RS;
                if (words) {
                    const uint32_t* s4 = reinterpret_cast<const uint32_t*>(src);
                    uint32_t* d4 = reinterpret_cast<uint32_t*>(dst);
                    for (int i = lane; i < (int)(RS * sizeof(T) / 4); i += 32) d4[i] = s4[i];
                } else {
                    for (int i = lane; i < RS; i += 32) dst[i] = src[i];
                }
            } else {
                for (int i = lane; i < RS; i += 32) dst[i] = from_f<T>(0.f);
            }
        }
        __syncthreads();
        if (!live) continue;
        // score of key (jt + lane)
        float s = 0.f;
        {
            const T* kr = tile + (long)lane * RSP;
            const float* a = qa + warp * R;
            const float* b = qr + warp * dr;
            if (sizeof(T) == 2 && !(R & 1) && !(dr & 1)) {     // two bf16 per 32-bit shared-memory load
                const uint32_t* k2 = reinterpret_cast<const uint32_t*>(kr);
                for (int d = 0; d < R; d += 2) {
                    const uint32_t w = k2[d >> 1];
                    const float2 q2 = *reinterpret_cast<const float2*>(a + d);
                    s = fmaf(q2.x, __uint_as_float(w << 16), s);
                    s = fmaf(q2.y, __uint_as_float(w & 0xffff0000u), s);
                }
                k2 += R >> 1;
                for (int d = 0; d < dr; d += 2) {
                    const uint32_t w = k2[d >> 1];
                    s = fmaf(b[d], __uint_as_float(w << 16), s);
                    s = fmaf(b[d + 1], __uint_as_float(w & 0xffff0000u), s);
                }
            } else {
                for (int d = 0; d < R; d++) s = fmaf(a[d], to_f(kr[d]), s);
                for (int d = 0; d < dr; d++) s = fmaf(b[d], to_f(kr[R + d]), s);
            }
        }
        s = (jt + lane < j1) ? s * p.scale : -INFINITY;
        const float mn = fmaxf(m, warp_max(s));
        const float corr = expf(m - mn);          // m = -inf only before the first tile, whose first key is always valid
        const float pj = expf(s - mn);
        l = l * corr + warp_sum(pj);
        m = mn;
        pw[warp * kWinTile + lane] = pj;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < NI; i++) acc[i] *= corr;
        const int nk = min(kWinTile, j1 - jt);
        for (int j = 0; j < nk; j++) {
            const float w = pw[warp * kWinTile + j];
            const T* kr = tile + (long)j * RSP;
            if (VW == 2) {
                const uint32_t* k2 = reinterpret_cast<const uint32_t*>(kr);
#pragma unroll
                for (int i = 0; i < NI / 2; i++) {
                    const int c = lane + 32 * i;              // column pair (2c, 2c + 1)
                    if (2 * c < R) {
                        const uint32_t u = k2[c];
                        acc[2 * i] = fmaf(w, __uint_as_float(u << 16), acc[2 * i]);
                        acc[2 * i + 1] = fmaf(w, __uint_as_float(u & 0xffff0000u), acc[2 * i + 1]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    const int d = lane + 32 * i;
                    if (d < R) acc[i] = fmaf(w, to_f(kr[d]), acc[i]);
                }
            }
        }
        __syncwarp();
    }
    if (!live) return;
    if (SPLIT) {
        float* o = p.part + (((long)t * p.H + h) * p.splits + blockIdx.z) * (R + 2);
        if (lane == 0) { o[0] = m; o[1] = l; }
#pragma unroll
        for (int i = 0; i < NI; i++) {
            const int d = col(i);
            if (d < R) o[2 + d] = acc[i];
        }
    } else {
        T* o = reinterpret_cast<T*>(p.out) + ((long)t * p.H + h) * R;
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < NI; i++) {
            const int d = col(i);
            if (d < R) o[d] = from_f<T>(acc[i] * inv);
        }
    }
}

// one CTA of 128 threads per (token, head): the parts' weights exp(m_s - m) / l once in shared memory (parts without a key
// have m = -inf and weight 0), the sink in the denominator, then the columns in parallel
template <typename T>
__global__ void __launch_bounds__(128) latent_window_merge_kernel(const WinAttnParams p) {
    __shared__ float wgt[64];
    __shared__ float red[4];
    const int w = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = w % p.H, R = p.R;
    const float* part = p.part + (long)w * p.splits * (R + 2);
    const float ms = tid < p.splits ? part[(long)tid * (R + 2)] : -INFINITY;        // splits <= 64
    const float ls = tid < p.splits ? part[(long)tid * (R + 2) + 1] : 0.f;
    float m = warp_max(ms);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    if (p.sink) m = fmaxf(m, p.sink[h]);
    __syncthreads();
    const float e = ms > -INFINITY ? expf(ms - m) : 0.f;
    float l = warp_sum(ls * e);
    if (lane == 0) red[warp] = l;
    __syncthreads();
    l = (red[0] + red[1]) + (red[2] + red[3]);
    if (p.sink) l += expf(p.sink[h] - m);
    if (tid < p.splits) wgt[tid] = e / l;
    __syncthreads();
    T* o = reinterpret_cast<T*>(p.out) + (long)w * R;
    for (int d = tid; d < R; d += 128) {
        float a = 0.f;
        for (int s = 0; s < p.splits; s++) a = fmaf(wgt[s], part[(long)s * (R + 2) + 2 + d], a);
        o[d] = from_f<T>(a);
    }
}

template <typename T, int NI>
static int launch_win(const WinAttnParams& p, size_t smem, cudaStream_t st) {
    const dim3 grid(p.T, (p.H + kWinWarps - 1) / kWinWarps, p.splits > 1 ? p.splits : 1);
    if (p.splits > 1) {
        static size_t granted = 48 * 1024;
        if (smem > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(latent_window_attn_kernel<T, NI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); granted = smem; }
        latent_window_attn_kernel<T, NI, true><<<grid, kWinWarps * 32, smem, st>>>(p);
        KTB_LAUNCH_CHECK();
        latent_window_merge_kernel<T><<<p.T * p.H, 128, 0, st>>>(p);
        KTB_LAUNCH_CHECK();
    } else {
        static size_t granted = 48 * 1024;
        if (smem > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(latent_window_attn_kernel<T, NI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); granted = smem; }
        latent_window_attn_kernel<T, NI, false><<<grid, kWinWarps * 32, smem, st>>>(p);
        KTB_LAUNCH_CHECK();
    }
    return KTB200_OK;
}
template <typename T>
static int launch_win_t(const WinAttnParams& p, size_t smem, cudaStream_t st) {
    const int ni = (p.R + 31) / 32;
    if (ni <= 4) return launch_win<T, 4>(p, smem, st);
    if (ni <= 8) return launch_win<T, 8>(p, smem, st);
    if (ni <= 16) return launch_win<T, 16>(p, smem, st);
    return launch_win<T, 32>(p, smem, st);
}

}  // namespace ktb

using namespace ktb;

extern "C" size_t ktb200_latent_window_attn_workspace(int n_tokens, int num_heads, int kv_rank, int splits) {
    return splits > 1 ? (size_t)n_tokens * num_heads * splits * (kv_rank + 2) * sizeof(float) : 0;
}

extern "C" int ktb200_latent_window_attn(const void* q, const void* q_abs, int num_heads, int dim, int rot_dim, int kv_rank, int rot_dims, int rot_layout, const double* inv_freq, float scale,
                                         const float* sink, int window, const int* pos, const int* slot, const int* page_table, int max_pages, int page_size, const void* cache,
                                         void* out, int n_tokens, int splits, void* workspace, int dtype, void* stream) {
    if (!q || !q_abs || !pos || !slot || !page_table || !cache || !out || num_heads <= 0 || dim < 0 || rot_dim < 0 || kv_rank <= 0 || kv_rank > 1024 || rot_dims < 0 ||
        rot_dims > rot_dim || (rot_dims & 1) || (rot_dims && !inv_freq) || (rot_layout != kRotInterleaved && rot_layout != kRotHalves) || max_pages <= 0 || page_size <= 0 || (splits > 1 && !workspace) || splits > 64) {
        set_error("latent_window_attn: bad argument (latent size <= 1024)");
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    const size_t esz = dtype == KTB200_TYPE_F32 ? 4 : 2;
    const int RS = kv_rank + rot_dim;
    int pad = 0;   // row stride of the shared-memory tile: an odd number of 32-bit words (bank-conflict-free column reads)
    while (((RS + pad) * esz) % 4 != 0 || (((RS + pad) * esz) / 4) % 2 == 0) pad++;
    const size_t smem = (size_t)kWinWarps * (kv_rank + rot_dim + kWinTile) * sizeof(float) + (size_t)kWinTile * (RS + pad) * esz;
    if (smem > 227 * 1024) { set_error("latent_window_attn: tile does not fit shared memory"); return KTB200_EINVAL; }
    WinAttnParams p{q, q_abs, inv_freq, sink, pos, slot, page_table, cache, out, (float*)workspace, n_tokens, num_heads, dim, rot_dim, kv_rank, rot_dims, rot_layout, window, max_pages,
                    page_size, pad, splits > 1 ? splits : 1, scale};
    if (dtype == KTB200_TYPE_BF16) return launch_win_t<__nv_bfloat16>(p, smem, (cudaStream_t)stream);
    if (dtype == KTB200_TYPE_F32) return launch_win_t<float>(p, smem, (cudaStream_t)stream);
    set_error("latent_window_attn: dtype must be bf16 or f32");
    return KTB200_EINVAL;
}
