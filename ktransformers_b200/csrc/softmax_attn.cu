// Soft-max attention over grouped key/value heads in a paged cache, with a partial rotation, normed queries and keys, capped
// scores, a sliding-window or chunked mask and values blended with another layer's (libktb200_seq.so).
//
//   ktb200_rope_norm_cache_write   proj rows [... q H*d ... k G*d ... v G*dv ...]: q and k turn over their first rot_dims columns (pairs of
//                                  either layout, angle pos * inv_freq[i]), then (qk_norm 1) are scaled to unit rms head by head, or
//                                  (qk_norm 2) divided by the rms of the WHOLE q (k) row and multiplied by a weight per column;
//                                  v <- (1 - t) v + t v_other with one learned t (optional), then each value head to unit rms (optional);
//                                  [k | v] into the paged cache, q into q_out
//   ktb200_window_softmax_attn     o_i = sum_j softmax_j(cap(scale t_h q_i.k_j)) v_j over the keys j <= i with i - j < window (window > 0)
//                                  and floor(j / chunk) == floor(i / chunk) (chunk > 0), cap(s) = c tanh(s / c), c = softcap (softcap <= 0:
//                                  none), t_h one learned number per query head (optional); query head h reads key/value head h / (H / G); the
//                                  key range is cut into splits for few tokens on long ranges; bf16 with head sizes that are multiples of 16
//                                  up to 128: m16n8k16 tensor-core tiles
//
// Storage type T (bf16 or float) for activations and cache rows; rotation, norms, scores, the cap and the soft-max are fp32
// (angles fp64).  Cache row of a token: [k G*d | v G*dv]; a sequence's page table row is a ring.
#include <cuda_bf16.h>

#include "common.cuh"
#include "seq_common.cuh"
#include "mma_tile.cuh"

namespace ktb {

// ------------------------------------------------------------------------------------------------ rotation, unit rms, value blend, cache write
// grid (tokens, unit blocks): a token's units are its H query heads, then its G key heads, then its G value heads; a CTA takes
// `units_per_cta` consecutive units, a warp per unit.  Prompt-sized batches run one CTA per token; small batches spread a token's units
// over several CTAs so that a decode step is not one warp's chain of heads.  What a CTA with query or key units needs of the whole
// token it computes itself: the rot_dims / 2 (cos, sin) pairs (fp64 angle and sincos, kept as fp32) and, for the row-wide norm, the
// sums of squares of the whole q row and the whole k row (16- / 8-byte loads where the rows allow them, one fixed order of addition).
constexpr int kPrepMaxPerLane = 8;      // head size <= 256
constexpr int kQkNormNone = 0, kQkNormHead = 1, kQkNormRow = 2;
template <typename T>
__device__ __forceinline__ float sum_squares(const T* __restrict__ x, int n, bool vec) {
    float s = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            const float4 v = load4(x + i);
            s += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f(x[i]); s += v * v; }
    }
    return s;
}
template <typename T>
__global__ void __launch_bounds__(256) rope_norm_cache_write_kernel(const T* __restrict__ proj, long proj_stride, int q_off, int k_off, int v_off, int H, int G, int d, int dv,
                                                                    int rot_dims, int rot_layout, const double* __restrict__ inv_freq, int qk_norm, const T* __restrict__ q_w,
                                                                    const T* __restrict__ k_w, int v_unit_rms, float eps, const T* __restrict__ v_other, long v_other_stride, const float* __restrict__ blend,
                                                                    const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ page_table,
                                                                    int max_pages, int page_size, T* __restrict__ cache, T* __restrict__ q_out, int units_per_cta, int vec_rows) {
    __shared__ float2 turn[16 * kPrepMaxPerLane];      // (cos, sin) of the token's angles
    __shared__ float red[8], row_inv[2];
    const long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int units = H + 2 * G, u0 = blockIdx.y * units_per_cta, u1 = min(units, u0 + units_per_cta);
    const int p = pos[t], half = rot_dims >> 1;
    const T* row = proj + t * proj_stride;
    if (u0 < H + G) {      // this CTA has query or key heads
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            double sn, cs;
            sincos((double)p * inv_freq[i], &sn, &cs);
            turn[i] = make_float2((float)cs, (float)sn);
        }
        if (qk_norm == kQkNormRow) {      // a turn keeps x^2 + y^2 of its pair: the row's mean square is that of the un-turned columns
            const float sq = block_sum(sum_squares(row + q_off, H * d, vec_rows), red);
            const float sk = block_sum(sum_squares(row + k_off, G * d, vec_rows), red);
            if (threadIdx.x == 0) {
                row_inv[0] = 1.0f / sqrtf(sq / (float)(H * d) + eps);
                row_inv[1] = 1.0f / sqrtf(sk / (float)(G * d) + eps);
            }
        }
        __syncthreads();
    }
    const long crow = ((long)page_table[(long)slot[t] * max_pages + (p / page_size) % max_pages] * page_size + p % page_size) * ((long)G * (d + dv));
    const float lam = v_other ? blend[0] : 0.f;
    for (int hh = u0 + warp; hh < min(u1, H + G); hh += nw) {
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
                if (i < rot_dims) {
                    const float other = to_f(src[rot_partner(i, rot_dims, rot_layout)]);
                    const bool second = rot_layout == kRotHalves ? i >= half : (i & 1);
                    const float2 cs = turn[rot_layout == kRotHalves ? (second ? i - half : i) : (i >> 1)];
                    v = second ? v * cs.x + other * cs.y : v * cs.x - other * cs.y;
                }
                r[e] = v;
                s += v * v;
            }
        }
        float inv = 1.f;
        if (qk_norm == kQkNormHead) {
            s = warp_sum(s);
            inv = 1.0f / sqrtf(s / (float)d + eps);
        } else if (qk_norm == kQkNormRow) {
            inv = row_inv[is_q ? 0 : 1];
        }
        T* dst = is_q ? q_out + (t * H + hh) * d : cache + crow + (long)(hh - H) * d;
        const T* wrow = qk_norm == kQkNormRow ? (is_q ? q_w + (long)hh * d : k_w + (long)(hh - H) * d) : nullptr;
#pragma unroll
        for (int e = 0; e < kPrepMaxPerLane; e++) {
            const int i = lane + 32 * e;
            if (i < d) dst[i] = from_f<T>(wrow ? r[e] * inv * to_f(wrow[i]) : r[e] * inv);
        }
    }
    // value heads: blend, mean square over the head's columns (optional), the scaled columns into the cache
    for (int hh = max(u0, H + G) + warp; hh < u1; hh += nw) {
        const int g = hh - H - G;
        const T* v = row + v_off + (long)g * dv;
        const T* vo = v_other ? v_other + t * v_other_stride + (long)g * dv : nullptr;
        T* dst = cache + crow + (long)G * d + (long)g * dv;
        float inv = 1.f;
        if (v_unit_rms) {
            float s = 0.f;
            for (int i = lane; i < dv; i += 32) {
                float x = to_f(v[i]);
                if (vo) x = (1.0f - lam) * x + lam * to_f(vo[i]);
                s += x * x;
            }
            inv = 1.0f / sqrtf(warp_sum(s) / (float)dv + eps);
        }
        for (int i = lane; i < dv; i += 32) {
            float x = to_f(v[i]);
            if (vo) x = (1.0f - lam) * x + lam * to_f(vo[i]);
            dst[i] = from_f<T>(v_unit_rms ? x * inv : x);
        }
    }
}

// ------------------------------------------------------------------------------------------------ soft-max attention, CUDA cores
// grid (tokens, G * head blocks, splits); a warp per query head (HB = blockDim / 32 heads of ONE key/value head per CTA).  Tiles of
// 32 keys in shared memory as fp32: lane = key for the scores, lane = value column for the weighted sum; running maximum and sum per
// warp.  Shared memory:  q [HB][d] | K [32][d + 1] | V [32][dv] | weights [HB][32]
constexpr int kSmTile = 32;
constexpr int kSmMaxCols = 8;      // value columns per lane: vdim <= 256
__device__ __forceinline__ float cap_score(float s, float softcap) { return softcap > 0.f ? softcap * tanhf(s / softcap) : s; }
// the first key that the query at position p sees: the start of its window, or of its chunk (chunks are counted from position 0)
__device__ __forceinline__ int first_visible(int p, int window, int chunk) {
    int lo = window > 0 ? max(0, p - window + 1) : 0;
    if (chunk > 0) lo = max(lo, p - p % chunk);
    return lo;
}

template <typename T>
__global__ void __launch_bounds__(256) window_softmax_attn_kernel(const T* __restrict__ q, int H, int G, int d, int dv, float scale, const float* __restrict__ head_scale,
                                                                  float softcap, int window, int chunk, const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ page_table,
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
    const int lo = first_visible(p, window, chunk), n_keys = p + 1 - lo;
    const int splits = gridDim.z;
    const int per = ((n_keys + splits - 1) / splits + kSmTile - 1) / kSmTile * kSmTile;
    const int k_lo = lo + blockIdx.z * per, k_hi = min(p + 1, k_lo + per);
    float acc[kSmMaxCols];
#pragma unroll
    for (int c = 0; c < kSmMaxCols; c++) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (k_lo < k_hi) {
        if (live) {
            const float sc = head_scale ? scale * head_scale[h] : scale;
            for (int i = lane; i < d; i += 32) qs[warp * d + i] = to_f(q[(t * H + h) * d + i]) * sc;
        }
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

// ------------------------------------------------------------------------------------------------ soft-max attention, tensor cores (bf16)
// A CTA of ROWS / 16 warps owns a tile of ROWS rows = (token, query head) pairs of ONE sequence portion and ONE key/value head: `RH`
// query heads of the group for each of ROWS / RH consecutive tokens (prompt portions fill the rows with tokens, decode steps with the
// group's heads, so grouped heads share every key tile).  Keys run in tiles of KEYS through a two-stage cp.async ring of [k | v]
// rows gathered through the page table, from the first key that the tile's earliest token still sees to its last token's own;
// S = Q K^T and O += P V are m16n8k16 bf16 MMAs with fp32 accumulators; scale, cap, window and causal masks, running maximum and
// sum in fp32 registers (a row's maximum over the four threads that hold it); the weights go to the second product as bf16.
// grid (tile bound, G * head blocks, splits); tiles are found from the per-sequence rows `seqs`.  Held to 128 registers (a few bytes of
// spills at head size 128) so that four CTAs share an SM: decode-shaped launches are bound by the copies in flight per SM.
constexpr int kMmaRows = 64, kMmaKeys = 32, kMmaPad = 8;
__device__ __forceinline__ float cap_score_fast(float s, float two_over_cap, float softcap) {
    // c tanh(s / c) as c (1 - 2 / (exp(2 s / c) + 1)), c = softcap: absolute error of a few 1e-7 of the cap
    return softcap * (1.0f - __fdividef(2.0f, __expf(s * two_over_cap) + 1.0f));
}

template <int D16MAX, int DV16MAX>
__global__ void __launch_bounds__(kMmaRows * 2, 4) window_softmax_attn_mma_kernel(
    const __nv_bfloat16* __restrict__ q, int H, int G, int d, int dv, float scale, const float* __restrict__ head_scale, float softcap, int window, int chunk,
    const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ seqs, int seqs_stride, int n_seqs, int RH, const int* __restrict__ page_table, int max_pages, int page_size, const __nv_bfloat16* __restrict__ cache,
    __nv_bfloat16* __restrict__ out, float* __restrict__ partial) {
    constexpr int ROWS = kMmaRows, KEYS = kMmaKeys;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int tile_info[3];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
    const int TOKS = ROWS / RH;
    if (tid == 0) {      // which sequence portion and which of its tokens this tile covers
        int b = blockIdx.x, found = -1, off = 0, len = 0;
        for (int s = 0; s < n_seqs; s++) {
            len = seqs[seqs_stride + s];
            const int nt = (len + TOKS - 1) / TOKS;
            if (b < nt) { found = s; off = b * TOKS; break; }
            b -= nt;
        }
        tile_info[0] = found;
        tile_info[1] = found >= 0 ? seqs[found] + off : 0;
        tile_info[2] = found >= 0 ? min(TOKS, len - off) : 0;
    }
    __syncthreads();
    if (tile_info[0] < 0) return;
    const int tok0 = tile_info[1], ntok = tile_info[2];
    const int R = H / G, hblocks = R / RH;
    const int g = blockIdx.y / hblocks, h0 = g * R + (blockIdx.y % hblocks) * RH;
    const int d16 = d >> 4, dv16 = dv >> 4, ldk = d + kMmaPad, ldv = dv + kMmaPad;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* Ks = Qs + ROWS * ldk;                     // [2][KEYS][ldk]
    __nv_bfloat16* Vs = Ks + 2 * KEYS * ldk;                 // [2][KEYS][ldv]
    const int pos0 = pos[tok0], max_pos = pos0 + ntok - 1;
    // the tile's key range [lo, max_pos], cut into this split's part in whole key tiles counted from lo
    const int lo = first_visible(pos0, window, chunk);
    const int splits = gridDim.z, n_keys = max_pos + 1 - lo;
    const int per = ((n_keys + splits - 1) / splits + KEYS - 1) / KEYS * KEYS;
    const int k_lo = lo + blockIdx.z * per, k_hi = min(max_pos + 1, k_lo + per);
    // this thread's two rows of the warp's 16
    const int rA = warp * 16 + gq, rB = rA + 8;
    const int tokA = rA / RH, tokB = rB / RH, hA = h0 + rA % RH, hB = h0 + rB % RH;
    const bool vA = tokA < ntok, vB = tokB < ntok;
    const int pA = pos0 + tokA, pB = pos0 + tokB;
    const int fA = first_visible(pA, window, chunk), fB = first_visible(pB, window, chunk);
    const float scA = head_scale ? scale * head_scale[hA] : scale, scB = head_scale ? scale * head_scale[hB] : scale;
    const bool warp_live = (warp * 16) / RH < ntok;
    const int warp_max_pos = pos0 + min(ntok - 1, (warp * 16 + 15) / RH), warp_min_pos = pos0 + (warp * 16) / RH;
    const int warp_first_key = first_visible(warp_min_pos, window, chunk);      // no row of this warp sees a key before this one
    const int warp_last_first = first_visible(warp_max_pos, window, chunk);    // every row of this warp sees the keys from here to its own
    const float two_over_cap = softcap > 0.f ? 2.0f / softcap : 0.f;
    float O[2 * DV16MAX][4];
#pragma unroll
    for (int n = 0; n < 2 * DV16MAX; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) O[n][e] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    if (k_lo < k_hi) {
        const int* pt = page_table + (long)slot[tok0] * max_pages;
        const long cw = (long)G * (d + dv);
        const int kc = d >> 3, vc = dv >> 3;      // 16-byte chunks per row
        for (int i = tid; i < ROWS * kc; i += blockDim.x) {
            const int r = i / kc, c = i - r * kc, tk = r / RH;
            const bool ok = tk < ntok;
            cp_async16(Qs + r * ldk + c * 8, ok ? q + ((long)(tok0 + tk) * H + h0 + r % RH) * d + c * 8 : q, ok);
        }
        // TPR neighbouring threads copy key row r of a tile: one page-table lookup per thread and tile, made a tile ahead of its copies
        constexpr int TPR = ROWS * 2 / KEYS;
        const int lrow = tid / TPR, lpar = tid % TPR;
        auto row_base = [&](int kp) -> long {
            return kp < k_hi ? ((long)pt[(kp / page_size) % max_pages] * page_size + kp % page_size) * cw : -1;
        };
        auto load_tile = [&](int stage, long base) {
            __nv_bfloat16* kd = Ks + stage * KEYS * ldk + lrow * ldk;
            __nv_bfloat16* vd = Vs + stage * KEYS * ldv + lrow * ldv;
            const bool ok = base >= 0;
            const __nv_bfloat16* ksrc = ok ? cache + base + (long)g * d : cache;
            const __nv_bfloat16* vsrc = ok ? cache + base + (long)G * d + (long)g * dv : cache;
            for (int c = lpar; c < kc; c += TPR) cp_async16(kd + c * 8, ok ? ksrc + c * 8 : cache, ok);
            for (int c = lpar; c < vc; c += TPR) cp_async16(vd + c * 8, ok ? vsrc + c * 8 : cache, ok);
        };
        load_tile(0, row_base(k_lo + lrow));
        long next_base = row_base(k_lo + KEYS + lrow);
        int stage = 0;
        for (int j0 = k_lo; j0 < k_hi; j0 += KEYS, stage ^= 1) {
            cp_async_wait_all();
            __syncthreads();      // this tile has landed, and every warp is done with the other stage
            if (j0 + KEYS < k_hi) {
                load_tile(stage ^ 1, next_base);
                next_base = row_base(j0 + 2 * KEYS + lrow);
            }
            if (!warp_live || j0 > warp_max_pos || j0 + KEYS <= warp_first_key) continue;
            const __nv_bfloat16* kt = Ks + stage * KEYS * ldk;
            const __nv_bfloat16* vt = Vs + stage * KEYS * ldv;
            float S[KEYS / 8][4];
#pragma unroll
            for (int n = 0; n < KEYS / 8; n++)
#pragma unroll
                for (int e = 0; e < 4; e++) S[n][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D16MAX; kk++) {
                if (kk < d16) {
                    uint32_t a[4];
                    ldmatrix_x4(a, Qs + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ldk + kk * 16 + 8 * (lane >> 4));
#pragma unroll
                    for (int np = 0; np < KEYS / 16; np++) {      // two key n-tiles per ldmatrix
                        uint32_t b[4];
                        ldmatrix_x4(b, kt + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * ldk + kk * 16 + 8 * ((lane >> 3) & 1));
                        mma_bf16_16816(S[2 * np], a, b[0], b[1]);
                        mma_bf16_16816(S[2 * np + 1], a, b[2], b[3]);
                    }
                }
            }
            // nothing to mask: all 16 rows carry tokens, and every key of the tile lies at or before the earliest of them, inside the
            // window or chunk of the latest and inside this split
            const bool plain = (warp * 16 + 15) / RH < ntok && j0 + KEYS - 1 <= warp_min_pos && j0 >= warp_last_first && j0 + KEYS <= k_hi;
            float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
            for (int n = 0; n < KEYS / 8; n++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float s = S[n][e] * (e < 2 ? scA : scB);
                    if (softcap > 0.f) s = cap_score_fast(s, two_over_cap, softcap);
                    if (!plain) {
                        const int key = j0 + n * 8 + 2 * tq + (e & 1);
                        const bool second = e >= 2;
                        const bool ok = (second ? vB : vA) && key <= (second ? pB : pA) && key >= (second ? fB : fA) && key < k_hi;
                        if (!ok) s = -INFINITY;
                    }
                    S[n][e] = s;
                    if (e < 2) tmA = fmaxf(tmA, s);
                    else tmB = fmaxf(tmB, s);
                }
            }
            tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1));
            tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
            tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1));
            tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
            const float nA = fmaxf(mA, tmA), nB = fmaxf(mB, tmB);
            const float uA = nA == -INFINITY ? 0.f : nA, uB = nB == -INFINITY ? 0.f : nB;      // a row that has seen no key yet keeps weights of zero
            const float cA = __expf(mA - uA), cB = __expf(mB - uB);
            mA = nA;
            mB = nB;
            float sA = 0.f, sB = 0.f;
#pragma unroll
            for (int n = 0; n < KEYS / 8; n++) {
                S[n][0] = __expf(S[n][0] - uA);
                S[n][1] = __expf(S[n][1] - uA);
                S[n][2] = __expf(S[n][2] - uB);
                S[n][3] = __expf(S[n][3] - uB);
                sA += S[n][0] + S[n][1];
                sB += S[n][2] + S[n][3];
            }
            lA = lA * cA + sA;
            lB = lB * cB + sB;
#pragma unroll
            for (int n = 0; n < 2 * DV16MAX; n++) {
                O[n][0] *= cA;
                O[n][1] *= cA;
                O[n][2] *= cB;
                O[n][3] *= cB;
            }
#pragma unroll
            for (int kk = 0; kk < KEYS / 16; kk++) {      // 16 keys per step
                uint32_t a[4] = {pack_bf16(S[2 * kk][0], S[2 * kk][1]), pack_bf16(S[2 * kk][2], S[2 * kk][3]), pack_bf16(S[2 * kk + 1][0], S[2 * kk + 1][1]),
                                 pack_bf16(S[2 * kk + 1][2], S[2 * kk + 1][3])};
#pragma unroll
                for (int vp = 0; vp < DV16MAX; vp++) {
                    if (vp < dv16) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ldv + vp * 16 + 8 * (lane >> 4));
                        mma_bf16_16816(O[2 * vp], a, b[0], b[1]);
                        mma_bf16_16816(O[2 * vp + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        cp_async_wait_all();
    }
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    if (partial) {      // [T][H][splits][dv + 2]: running maximum, sum, un-normalised weighted values
        float* oA = partial + (((long)(tok0 + tokA) * H + hA) * splits + blockIdx.z) * (dv + 2);
        float* oB = partial + (((long)(tok0 + tokB) * H + hB) * splits + blockIdx.z) * (dv + 2);
        if (tq == 0) {
            if (vA) { oA[0] = mA; oA[1] = lA; }
            if (vB) { oB[0] = mB; oB[1] = lB; }
        }
#pragma unroll
        for (int n = 0; n < 2 * DV16MAX; n++) {
            const int col = n * 8 + 2 * tq;
            if (col < dv) {
                if (vA) *reinterpret_cast<float2*>(oA + 2 + col) = make_float2(O[n][0], O[n][1]);
                if (vB) *reinterpret_cast<float2*>(oB + 2 + col) = make_float2(O[n][2], O[n][3]);
            }
        }
    } else {
        const float iA = vA ? 1.0f / lA : 0.f, iB = vB ? 1.0f / lB : 0.f;
#pragma unroll
        for (int n = 0; n < 2 * DV16MAX; n++) {
            const int col = n * 8 + 2 * tq;
            if (col < dv) {
                if (vA) *reinterpret_cast<uint32_t*>(out + ((long)(tok0 + tokA) * H + hA) * dv + col) = pack_bf16(O[n][0] * iA, O[n][1] * iA);
                if (vB) *reinterpret_cast<uint32_t*>(out + ((long)(tok0 + tokB) * H + hB) * dv + col) = pack_bf16(O[n][2] * iB, O[n][3] * iB);
            }
        }
    }
}

// one CTA of 128 threads per (token, head): the parts' weights exp(m_s - m) / l once in shared memory (parts without a key have
// m = -inf and weigh nothing), then the columns in parallel, parts in order
constexpr int kMergeMaxSplits = 128;
template <typename T>
__global__ void __launch_bounds__(128) softmax_merge_kernel(const float* __restrict__ partial, int splits, T* __restrict__ out, int dv) {
    __shared__ float wgt[kMergeMaxSplits];
    __shared__ float red[4];
    const long row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* part = partial + row * splits * (dv + 2);
    const float ms = tid < splits ? part[(long)tid * (dv + 2)] : -INFINITY;
    const float ls = tid < splits ? part[(long)tid * (dv + 2) + 1] : 0.f;
    float m = warp_max(ms);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    const float e = ms > -INFINITY ? expf(ms - m) : 0.f;
    float l = warp_sum(ls * e);
    if (lane == 0) red[warp] = l;
    __syncthreads();
    l = (red[0] + red[1]) + (red[2] + red[3]);
    if (tid < splits) wgt[tid] = e / l;
    __syncthreads();
    for (int c = tid; c < dv; c += 128) {
        float a = 0.f;
        for (int s = 0; s < splits; s++) a = fmaf(wgt[s], part[(long)s * (dv + 2) + 2 + c], a);
        out[row * dv + c] = from_f<T>(a);
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
                                            int rot_layout, const double* inv_freq, int qk_norm, const void* q_weight, const void* k_weight, int v_unit_rms, float eps,
                                            const void* v_other, long v_other_stride, const float* blend, const int* pos, const int* slot, const int* page_table, int max_pages, int page_size, void* cache, void* q_out, int n_tokens,
                                            int dtype, void* stream) {
    if (!proj || !pos || !slot || !page_table || !cache || !q_out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim > 32 * kPrepMaxPerLane || vdim <= 0 ||
        rot_dims < 0 || rot_dims > dim || (rot_dims & 1) || (rot_dims && !inv_freq) || (rot_layout != kRotInterleaved && rot_layout != kRotHalves) || (v_other && !blend) ||
        qk_norm < kQkNormNone || qk_norm > kQkNormRow || (qk_norm == kQkNormRow && (!q_weight || !k_weight)) || page_size <= 0 || max_pages <= 0) {
        set_error("rope_norm_cache_write: bad argument (head size <= %d)", 32 * kPrepMaxPerLane);
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    // unit blocks per token: as many as keep about a wave of CTAs (148 SMs x 8) busy, eight units (one per warp) at least
    const int units = heads + 2 * kv_heads, max_y = (units + 7) / 8;
    int want_y = 1184 / n_tokens;
    want_y = want_y < 1 ? 1 : (want_y > max_y ? max_y : want_y);
    const int upc = ((units + want_y - 1) / want_y + 7) / 8 * 8, grid_y = (units + upc - 1) / upc;
    const size_t esz = dtype == KTB200_TYPE_BF16 ? 2 : 4;
    const int vec_rows = q_off % 4 == 0 && k_off % 4 == 0 && (heads * dim) % 4 == 0 && (kv_heads * dim) % 4 == 0 && proj_stride % 4 == 0 &&
                         (reinterpret_cast<uintptr_t>(proj) & (4 * esz - 1)) == 0;
    SEQ_DISPATCH(dtype, (rope_norm_cache_write_kernel<T><<<dim3(n_tokens, grid_y), 256, 0, (cudaStream_t)stream>>>(
                            (const T*)proj, proj_stride, q_off, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, rot_layout, inv_freq, qk_norm, (const T*)q_weight, (const T*)k_weight, v_unit_rms, eps,
                            (const T*)v_other, v_other_stride, blend, pos, slot, page_table, max_pages, page_size, (T*)cache, (T*)q_out, upc, vec_rows)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" size_t ktb200_window_softmax_attn_workspace(int n_tokens, int heads, int vdim, int splits) {
    return splits > 1 ? (size_t)n_tokens * heads * splits * (vdim + 2) * sizeof(float) : 0;
}

/* whether ktb200_window_softmax_attn runs tensor-core tiles for these sizes (bf16, head sizes multiples of 16 up to 128, and
 * `seqs` given), and an upper bound of its row tiles per key/value head (for choosing splits) */
extern "C" int ktb200_window_softmax_attn_uses_tensor_cores(int heads, int kv_heads, int dim, int vdim, int dtype) {
    return dtype == KTB200_TYPE_BF16 && kv_heads > 0 && heads % kv_heads == 0 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 128 && vdim <= 128;
}
extern "C" int ktb200_window_softmax_attn_tiles(int heads, int kv_heads, int n_tokens, int n_seqs) {
    return n_seqs + n_tokens / (kMmaRows / mma_heads_per_tile(heads / kv_heads));
}

extern "C" int ktb200_window_softmax_attn(const void* q, int heads, int kv_heads, int dim, int vdim, float scale, const float* head_scale, float softcap, int window, int chunk,
                                          const int* pos, const int* slot,
                                          const int* seqs, int seqs_stride, int n_seqs, const int* page_table, int max_pages, int page_size, const void* cache, void* out,
                                          int n_tokens, int splits, float* workspace, int dtype, int allow_tensor_cores, void* stream) {
    if (!q || !pos || !slot || !page_table || !cache || !out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || vdim > 32 * kSmMaxCols ||
        splits < 1 || (splits > 1 && !workspace) || page_size <= 0 || max_pages <= 0) {
        set_error("window_softmax_attn: bad argument (value size <= %d)", 32 * kSmMaxCols);
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    if (splits > kMergeMaxSplits) { set_error("window_softmax_attn: at most %d splits", kMergeMaxSplits); return KTB200_EINVAL; }
    const long rows = (long)n_tokens * heads;
    if (allow_tensor_cores && seqs && n_seqs > 0 && ktb200_window_softmax_attn_uses_tensor_cores(heads, kv_heads, dim, vdim, dtype)) {
        using B = __nv_bfloat16;
        const int RH = mma_heads_per_tile(heads / kv_heads);
        const dim3 grid(ktb200_window_softmax_attn_tiles(heads, kv_heads, n_tokens, n_seqs), kv_heads * (heads / kv_heads / RH), splits);
        const size_t smem = (((size_t)kMmaRows + 2 * kMmaKeys) * (dim + kMmaPad) + (size_t)2 * kMmaKeys * (vdim + kMmaPad)) * sizeof(B);
#define MMA_LAUNCH(DK, DV)                                                                                                                                      \
    do {                                                                                                                                                        \
        GRANT_SMEM((window_softmax_attn_mma_kernel<DK, DV>), smem);                                                                                             \
        window_softmax_attn_mma_kernel<DK, DV><<<grid, kMmaRows * 2, smem, (cudaStream_t)stream>>>((const B*)q, heads, kv_heads, dim, vdim, scale, head_scale, softcap, window, chunk, pos, slot, \
                                                                                                   seqs, seqs_stride, n_seqs, RH, page_table, max_pages, page_size,  \
                                                                                                   (const B*)cache, (B*)out, splits > 1 ? workspace : nullptr);   \
    } while (0)
        if (dim <= 64 && vdim <= 64) MMA_LAUNCH(4, 4);
        else MMA_LAUNCH(8, 8);
#undef MMA_LAUNCH
        KTB_LAUNCH_CHECK();
        if (splits > 1) {
            softmax_merge_kernel<B><<<(unsigned)rows, 128, 0, (cudaStream_t)stream>>>(workspace, splits, (B*)out, vdim);
            KTB_LAUNCH_CHECK();
        }
        return KTB200_OK;
    }
    const int R = heads / kv_heads, HB = R < 8 ? R : 8, hblocks = (R + HB - 1) / HB;
    const size_t smem = ((size_t)HB * dim + (size_t)kSmTile * (dim + 1) + (size_t)kSmTile * vdim + (size_t)HB * kSmTile) * sizeof(float);
    if (smem > 200 * 1024) { set_error("window_softmax_attn: head too wide for shared memory"); return KTB200_EINVAL; }
    SEQ_DISPATCH(dtype, {
        GRANT_SMEM(window_softmax_attn_kernel<T>, smem);
        window_softmax_attn_kernel<T><<<dim3(n_tokens, kv_heads * hblocks, splits), HB * 32, smem, (cudaStream_t)stream>>>(
            (const T*)q, heads, kv_heads, dim, vdim, scale, head_scale, softcap, window, chunk, pos, slot, page_table, max_pages, page_size, (const T*)cache, (T*)out,
            splits > 1 ? workspace : nullptr, n_tokens);
        KTB_LAUNCH_CHECK();
        if (splits > 1) {
            softmax_merge_kernel<T><<<(unsigned)rows, 128, 0, (cudaStream_t)stream>>>(workspace, splits, (T*)out, vdim);
            KTB_LAUNCH_CHECK();
        }
    });
    return KTB200_OK;
}
