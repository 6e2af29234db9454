// Token-major operators of decoder layers with norms on both sides of every sublayer, sigmoid (un-normalised) attention with
// a distance bias, and gated linear attention with a recurrent state (libktb200_seq.so).
//
//   ktb200_group_rmsnorm_sandwich  x_out = x_in + gnorm(y) * (w_post + c) + row   then   h = gnorm(x_out) * (w_pre + c)
//                                  (gnorm: RMS norm in `groups` equal consecutive parts; every term optional; c = 0, or 1 for
//                                  zero-centred weights; without w_pre, h is x_out rounded to the compute dtype)
//   ktb200_qk_norm_cache_write     per-head RMS norm of queries and keys, query temperature by position, paged write of [k | v]
//   ktb200_sigmoid_bias_attn       o_i = sum_{j <= i} sigmoid(scale q_i.k_j + bias[h][min(i - j, n - 1)] + pb[h]) v_j over the paged
//                                  cache, grouped query heads, times sigmoid(gate[i][h]); key range cut into splits for few tokens;
//                                  bf16 with head sizes that are multiples of 16 up to 128: m16n8k16 tensor-core tiles
//   ktb200_gla_scan                S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per sequence portion, state rows in fp32,
//                                  a_t = sigmoid(z_t + b)^(1/tau)
//   ktb200_gla_out                 per-head RMS norm of o times silu(gate)
//   ktb200_xielu                   z > 0: sp(p) z^2 + z/2 ;  z <= 0: (1/2 + sp(q)) (exp(z) - 1 - z) + z/2 ,  sp = softplus
//   ktb200_gated_act_mul           gated activation of (gate, up) rows: SiLU or tanh-GELU of the gate times up, or the clamped sigmoid form
//   ktb200_relu_squared            relu(z)^2
//   ktb200_softcap                 c tanh(z / c) into fp32
//
// Storage type T (bf16 or float) for activations, weights and cache rows; every sum, norm, score, weight, decay and state is
// fp32.  Rows are addressed through per-token / per-sequence index arrays: one launch serves a ragged batch.
#include <cuda_bf16.h>

#include "common.cuh"
#include "seq_common.cuh"
#include "mma_tile.cuh"

namespace ktb {

__device__ __forceinline__ float sigmoid_f(float x) { return __fdiv_rn(1.0f, 1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
// log(sigmoid(x)) without overflow on either side
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ void prefetch_l2_line(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// ------------------------------------------------------------------------------------------------ sandwich norm
// One CTA per token.  Shared memory: red[32] | row[D] (the new residual row, when it fits).
template <typename T>
__global__ void __launch_bounds__(256) sandwich_norm_kernel(const float* __restrict__ x_in, const void* __restrict__ y, int y_type, const T* __restrict__ w_post,
                                                            const float* __restrict__ row_add, float* __restrict__ x_out, const T* __restrict__ w_pre,
                                                            T* __restrict__ h_out, int groups, float eps, int D, int stash, float w_off) {
    extern __shared__ __align__(16) float sm[];
    float* red = sm;
    float* row = sm + 32;
    const long t = blockIdx.x;
    const int tid = threadIdx.x, gs = D / groups;
    const bool vec = (gs & 3) == 0;
    const int lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    if (stash && nw % groups == 0 && gs % (4 * (nw / groups)) == 0) {
        // every warp owns one of nw equal chunks of the row (a group = nw / groups consecutive chunks): all groups advance together,
        // three barriers per row, 16-byte accesses; what the later passes read is asked into L2 while the first pass runs
        const int per = nw / groups, chunk = gs / per, lo = warp * chunk, g0 = (warp / per) * per;
        for (int i = lane * 32; i < chunk; i += 1024) {
            if (x_in) prefetch_l2_line(x_in + t * D + lo + i);
            if (row_add) prefetch_l2_line(row_add + lo + i);
        }
        for (int i = lane * (128 / (int)sizeof(T)); i < chunk; i += 32 * (128 / (int)sizeof(T))) {
            if (w_post) prefetch_l2_line(w_post + lo + i);
            if (w_pre) prefetch_l2_line(w_pre + lo + i);
        }
        float s = 0.f;
        for (int i = lane * 4; i < chunk; i += 128) {
            const float4 v = load4_hidden(y, t * D + lo + i, y_type);
            store4(row + lo + i, v);
            s += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        float inv = 1.f;
        if (w_post) {
            s = warp_sum(s);
            if (lane == 0) red[warp] = s;
            __syncthreads();
            float a = 0.f;
            for (int k = 0; k < per; k++) a += red[g0 + k];
            inv = 1.0f / sqrtf(a / (float)gs + eps);
        }
        float s2 = 0.f;
        for (int i = lane * 4; i < chunk; i += 128) {
            float4 v = load4(row + lo + i);
            if (w_post) { const float4 w = load4(w_post + lo + i); v.x = v.x * inv * (w.x + w_off); v.y = v.y * inv * (w.y + w_off); v.z = v.z * inv * (w.z + w_off); v.w = v.w * inv * (w.w + w_off); }
            if (x_in) { const float4 u = load4(x_in + t * D + lo + i); v.x = u.x + v.x; v.y = u.y + v.y; v.z = u.z + v.z; v.w = u.w + v.w; }
            if (row_add) { const float4 u = load4(row_add + lo + i); v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w; }
            if (x_out) store4(x_out + t * D + lo + i, v);
            if (h_out && !w_pre) store4(h_out + t * D + lo + i, v);      // the next sublayer reads the residual itself
            store4(row + lo + i, v);
            s2 += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        if (w_pre) {
            s2 = warp_sum(s2);
            if (lane == 0) red[16 + warp] = s2;
            __syncthreads();
            float a = 0.f;
            for (int k = 0; k < per; k++) a += red[16 + g0 + k];
            const float inv2 = 1.0f / sqrtf(a / (float)gs + eps);
            for (int i = lane * 4; i < chunk; i += 128) {
                float4 v = load4(row + lo + i);
                const float4 w = load4(w_pre + lo + i);
                v.x = v.x * inv2 * (w.x + w_off); v.y = v.y * inv2 * (w.y + w_off); v.z = v.z * inv2 * (w.z + w_off); v.w = v.w * inv2 * (w.w + w_off);
                store4(h_out + t * D + lo + i, v);
            }
        }
        return;
    }
    for (int g = 0; g < groups; g++) {
        const int lo = g * gs;
        float inv = 1.f;
        if (w_post) {
            float s = 0.f;
            if (vec) {
                for (int i = tid * 4; i < gs; i += blockDim.x * 4) {
                    const float4 v = load4_hidden(y, t * D + lo + i, y_type);
                    s += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
                }
            } else {
                for (int i = tid; i < gs; i += blockDim.x) { const float v = load_hidden(y, t * D + lo + i, y_type); s += v * v; }
            }
            s = block_sum(s, red);
            inv = 1.0f / sqrtf(s / (float)gs + eps);
        }
        float s2 = 0.f;
        for (int i = tid; i < gs; i += blockDim.x) {
            const long at = t * D + lo + i;
            float v = load_hidden(y, at, y_type);
            if (w_post) v = v * inv * (to_f(w_post[lo + i]) + w_off);
            if (x_in) v = x_in[at] + v;
            if (row_add) v += row_add[lo + i];
            if (x_out) x_out[at] = v;
            if (h_out && !w_pre) h_out[at] = from_f<T>(v);
            if (stash) row[lo + i] = v;
            s2 += v * v;
        }
        if (w_pre) {
            s2 = block_sum(s2, red);
            const float inv2 = 1.0f / sqrtf(s2 / (float)gs + eps);
            for (int i = tid; i < gs; i += blockDim.x) {      // the same thread wrote these values
                const float v = stash ? row[lo + i] : x_out[t * D + lo + i];
                h_out[t * D + lo + i] = from_f<T>(v * inv2 * (to_f(w_pre[lo + i]) + w_off));
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ attention: norms, temperature, cache write
// One CTA per token, a warp per head.  proj row: [q H*d | k G*d | v G*dv | ...].  Cache row: [k G*d | v G*dv].
template <typename T>
__global__ void __launch_bounds__(256) qk_norm_cache_write_kernel(const T* __restrict__ proj, long proj_stride, int H, int G, int d, int dv, const T* __restrict__ qw,
                                                                  const T* __restrict__ kw, float eps, float temp_coef, int temp_every, const int* __restrict__ pos,
                                                                  const int* __restrict__ slot, const int* __restrict__ page_table, int max_pages, int page_size,
                                                                  T* __restrict__ cache, T* __restrict__ q_out) {
    const long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int p = pos[t];
    const float temp = 1.0f + temp_coef * logf((float)((p + 1) / temp_every) + 1.0f);
    const T* row = proj + t * proj_stride;
    const long crow = ((long)page_table[(long)slot[t] * max_pages + (p / page_size) % max_pages] * page_size + p % page_size) * ((long)G * (d + dv));
    for (int hh = warp; hh < H + G; hh += nw) {
        const bool is_q = hh < H;
        const T* src = row + (long)hh * d;
        float s = 0.f;
        for (int i = lane; i < d; i += 32) { const float v = to_f(src[i]); s += v * v; }
        s = warp_sum(s);
        const float inv = 1.0f / sqrtf(s / (float)d + eps);
        if (is_q) {
            for (int i = lane; i < d; i += 32) q_out[(t * H + hh) * d + i] = from_f<T>(to_f(src[i]) * inv * to_f(qw[i]) * temp);
        } else {
            for (int i = lane; i < d; i += 32) cache[crow + (long)(hh - H) * d + i] = from_f<T>(to_f(src[i]) * inv * to_f(kw[i]));
        }
    }
    const T* v = row + (long)(H + G) * d;
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x) cache[crow + (long)G * d + i] = v[i];
}

// ------------------------------------------------------------------------------------------------ sigmoid attention, CUDA cores
// grid (tokens, G * head blocks, splits); a warp per query head (HB = blockDim / 32 heads of ONE key/value head per CTA).  Tiles of
// 32 keys in shared memory as fp32: lane = key for the scores, lane = value column for the weighted sum.  Shared memory:
//   q [HB][d] | K [32][d + 1] | V [32][dv] | bias [HB][n_bias]
constexpr int kAttnTile = 32;
constexpr int kAttnMaxCols = 8;      // value columns per lane: vdim <= 256
template <typename T>
__global__ void __launch_bounds__(256) sigmoid_attn_kernel(const T* __restrict__ q, int H, int G, int d, int dv, float scale, const float* __restrict__ bias, int n_bias,
                                                           const float* __restrict__ pb, const int* __restrict__ pos, const int* __restrict__ slot,
                                                           const int* __restrict__ page_table, int max_pages, int page_size, const T* __restrict__ cache,
                                                           const T* __restrict__ gate, long gate_stride, T* __restrict__ out, float* __restrict__ partial, int n_tokens, int stage_bias) {
    extern __shared__ __align__(16) float sm[];
    const int HB = blockDim.x >> 5, R = H / G, hblocks = (R + HB - 1) / HB;
    const int g = blockIdx.y / hblocks, hb = blockIdx.y % hblocks;
    const long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = hb * HB + warp, h = g * R + r;
    const bool live = r < R;
    float* qs = sm;
    float* Ks = qs + HB * d;
    float* Vs = Ks + kAttnTile * (d + 1);
    float* bs = Vs + kAttnTile * dv;
    const int p = pos[t];
    // key range of this split
    const int splits = gridDim.z, n_keys = p + 1;
    const int per = ((n_keys + splits - 1) / splits + kAttnTile - 1) / kAttnTile * kAttnTile;
    const int k_lo = blockIdx.z * per, k_hi = min(n_keys, k_lo + per);
    float acc[kAttnMaxCols];
#pragma unroll
    for (int c = 0; c < kAttnMaxCols; c++) acc[c] = 0.f;
    if (k_lo < k_hi) {
        if (live) {
            for (int i = lane; i < d; i += 32) qs[warp * d + i] = to_f(q[(t * H + h) * d + i]) * scale;
            if (stage_bias)      // a head's bias by distance, when the tables fit shared memory; read from global memory otherwise
                for (int i = lane; i < n_bias; i += 32) bs[warp * n_bias + i] = bias[(long)h * n_bias + i] + pb[h];
        }
        const int* pt = page_table + (long)slot[t] * max_pages;
        const long cw = (long)G * (d + dv);
        for (int j0 = k_lo; j0 < k_hi; j0 += kAttnTile) {
            __syncthreads();
            const int nk = min(kAttnTile, k_hi - j0);
            for (int i = threadIdx.x; i < nk * d; i += blockDim.x) {
                const int j = i / d, c = i - j * d, kp = j0 + j;
                Ks[j * (d + 1) + c] = to_f(cache[((long)pt[(kp / page_size) % max_pages] * page_size + kp % page_size) * cw + (long)g * d + c]);
            }
            for (int i = threadIdx.x; i < nk * dv; i += blockDim.x) {
                const int j = i / dv, c = i - j * dv, kp = j0 + j;
                Vs[j * dv + c] = to_f(cache[((long)pt[(kp / page_size) % max_pages] * page_size + kp % page_size) * cw + (long)G * d + (long)g * dv + c]);
            }
            __syncthreads();
            if (live) {
                float w = 0.f;
                if (lane < nk) {
                    float s = 0.f;
                    const float* kr = Ks + lane * (d + 1);
                    const float* qr = qs + warp * d;
                    for (int i = 0; i < d; i++) s = fmaf(qr[i], kr[i], s);
                    const int dist = p - (j0 + lane);
                    const int bi = min(dist, n_bias - 1);
                    w = sigmoid_f(s + (stage_bias ? bs[warp * n_bias + bi] : bias[(long)h * n_bias + bi] + pb[h]));
                }
                for (int j = 0; j < nk; j++) {
                    const float wj = __shfl_sync(0xffffffffu, w, j);
#pragma unroll
                    for (int c = 0; c < kAttnMaxCols; c++)
                        if (lane + 32 * c < dv) acc[c] = fmaf(wj, Vs[j * dv + lane + 32 * c], acc[c]);
                }
            }
        }
    }
    if (!live) return;
    if (partial) {
#pragma unroll
        for (int c = 0; c < kAttnMaxCols; c++)
            if (lane + 32 * c < dv) partial[(((long)blockIdx.z * n_tokens + t) * H + h) * dv + lane + 32 * c] = acc[c];
    } else {
        const float gt = sigmoid_f(to_f(gate[t * gate_stride + h]));
#pragma unroll
        for (int c = 0; c < kAttnMaxCols; c++)
            if (lane + 32 * c < dv) out[(t * H + h) * dv + lane + 32 * c] = from_f<T>(acc[c] * gt);
    }
}

// ------------------------------------------------------------------------------------------------ sigmoid attention, tensor cores (bf16)
// A CTA of ROWS / 16 warps owns a tile of ROWS (64 as launched) rows = (token, query head) pairs of ONE sequence portion and ONE
// key/value head: `RH` query heads of the group for each of ROWS / RH consecutive tokens; KEYS (32 as launched) keys per ring stage (prompt portions fill the rows with tokens, decode steps with the
// group's heads).  Keys run in tiles of KEYS through a two-stage cp.async ring of [k | v] rows gathered through the page table;
// S = Q K^T and O += P V are m16n8k16 bf16 MMAs with fp32 accumulators; the scores are scaled, biased and pushed through the
// sigmoid in fp32 registers and handed to the second product as bf16.  No running maximum and no rescaling: the weights are
// not normalised.  grid (tile bound, G * head blocks, splits); tiles are found from the per-sequence rows `seqs`.
constexpr int kMmaRows = 64, kMmaKeys = 64, kMmaPad = 8;

__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

template <int D16MAX, int DV16MAX, int ROWS, int KEYS>
__global__ void __launch_bounds__(ROWS * 2, (ROWS == 64 && KEYS == 32) ? 4 : 1) sigmoid_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, int H, int G, int d, int dv, float scale, const float* __restrict__ biasT,
                                                               int n_bias, const float* __restrict__ pb, const int* __restrict__ pos, const int* __restrict__ slot,
                                                               const int* __restrict__ seqs, int seqs_stride, int n_seqs, int RH, const int* __restrict__ page_table,
                                                               int max_pages, int page_size, const __nv_bfloat16* __restrict__ cache,
                                                               const __nv_bfloat16* __restrict__ gate, long gate_stride, __nv_bfloat16* __restrict__ out,
                                                               float* __restrict__ partial, int n_tokens) {
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
    __nv_bfloat16* Ks = Qs + ROWS * ldk;                 // [2][KEYS][ldk]
    __nv_bfloat16* Vs = Ks + 2 * KEYS * ldk;                 // [2][KEYS][ldv]
    const int pos0 = pos[tok0], max_pos = pos0 + ntok - 1;
    const int splits = gridDim.z, n_keys = max_pos + 1;
    const int per = ((n_keys + splits - 1) / splits + kMmaKeys - 1) / kMmaKeys * kMmaKeys;
    const int k_lo = blockIdx.z * per, k_hi = min(n_keys, k_lo + per);
    // this thread's two rows of the warp's 16
    const int rA = warp * 16 + gq, rB = rA + 8;
    const int tokA = rA / RH, tokB = rB / RH, hA = h0 + rA % RH, hB = h0 + rB % RH;
    const bool vA = tokA < ntok, vB = tokB < ntok;
    const int pA = pos0 + tokA, pB = pos0 + tokB;
    const bool warp_live = (warp * 16) / RH < ntok;
    const int warp_max_pos = pos0 + min(ntok - 1, (warp * 16 + 15) / RH), warp_min_pos = pos0 + (warp * 16) / RH;
    float O[2 * DV16MAX][4];
#pragma unroll
    for (int n = 0; n < 2 * DV16MAX; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) O[n][e] = 0.f;
    if (k_lo < k_hi) {
        const int* pt = page_table + (long)slot[tok0] * max_pages;
        const long cw = (long)G * (d + dv);
        const int kc = d >> 3, vc = dv >> 3;      // 16-byte chunks per row
        for (int i = tid; i < ROWS * kc; i += blockDim.x) {
            const int r = i / kc, c = i - r * kc, tk = r / RH;
            const bool ok = tk < ntok;
            cp_async16(Qs + r * ldk + c * 8, ok ? q + ((long)(tok0 + tk) * H + h0 + r % RH) * d + c * 8 : q, ok);
        }
        // TPR = 2 or 4 neighbouring threads copy key row r of a tile: one page-table lookup per thread and tile, made a tile ahead
        // of its copies, and 16-byte chunks dealt out over the TPR threads (together they fill whole 32-byte sectors)
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
        const float* bA = biasT + (long)hA * n_bias;
        const float* bB = biasT + (long)hB * n_bias;
        const float pbA = pb[hA], pbB = pb[hB];
        const float farA = bA[n_bias - 1] + pbA, farB = bB[n_bias - 1] + pbB;
        int stage = 0;
        for (int j0 = k_lo; j0 < k_hi; j0 += KEYS, stage ^= 1) {
            cp_async_wait_all();
            __syncthreads();      // this tile has landed, and every warp is done with the other stage
            if (j0 + KEYS < k_hi) {
                load_tile(stage ^ 1, next_base);
                next_base = row_base(j0 + 2 * KEYS + lrow);
            }
            if (!warp_live || j0 > warp_max_pos) continue;
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
            const bool far = warp_min_pos - (j0 + KEYS - 1) >= n_bias - 1;      // every distance of this warp's rows in this tile reads the table's last entry
            // and nothing to mask: all 16 rows carry tokens, every key of the tile lies at or before the earliest of them and inside this split
            const bool plain = far && (warp * 16 + 15) / RH < ntok && j0 + KEYS <= k_hi;
            if (plain) {
#pragma unroll
                for (int n = 0; n < KEYS / 8; n++) {
                    S[n][0] = sigmoid_fast(fmaf(S[n][0], scale, farA));
                    S[n][1] = sigmoid_fast(fmaf(S[n][1], scale, farA));
                    S[n][2] = sigmoid_fast(fmaf(S[n][2], scale, farB));
                    S[n][3] = sigmoid_fast(fmaf(S[n][3], scale, farB));
                }
            } else {
#pragma unroll
                for (int n = 0; n < KEYS / 8; n++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int key = j0 + n * 8 + 2 * tq + (e & 1);
                        const bool second = e >= 2;
                        const int dist = (second ? pB : pA) - key;
                        const bool ok = (second ? vB : vA) && dist >= 0 && key < k_hi;
                        float bias_v = second ? farB : farA;
                        if (!far && ok) bias_v = __ldg((second ? bB : bA) + min(dist, n_bias - 1)) + (second ? pbB : pbA);
                        S[n][e] = ok ? sigmoid_fast(fmaf(S[n][e], scale, bias_v)) : 0.f;
                    }
                }
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
    const float gA = (vA && !partial) ? sigmoid_f(__bfloat162float(gate[(long)(tok0 + tokA) * gate_stride + hA])) : 0.f;
    const float gB = (vB && !partial) ? sigmoid_f(__bfloat162float(gate[(long)(tok0 + tokB) * gate_stride + hB])) : 0.f;
#pragma unroll
    for (int n = 0; n < 2 * DV16MAX; n++) {
        const int col = n * 8 + 2 * tq;
        if (col < dv) {
            if (partial) {
                if (vA) *reinterpret_cast<float2*>(partial + (((long)blockIdx.z * n_tokens + tok0 + tokA) * H + hA) * dv + col) = make_float2(O[n][0], O[n][1]);
                if (vB) *reinterpret_cast<float2*>(partial + (((long)blockIdx.z * n_tokens + tok0 + tokB) * H + hB) * dv + col) = make_float2(O[n][2], O[n][3]);
            } else {
                if (vA) *reinterpret_cast<uint32_t*>(out + ((long)(tok0 + tokA) * H + hA) * dv + col) = pack_bf16(O[n][0] * gA, O[n][1] * gA);
                if (vB) *reinterpret_cast<uint32_t*>(out + ((long)(tok0 + tokB) * H + hB) * dv + col) = pack_bf16(O[n][2] * gB, O[n][3] * gB);
            }
        }
    }
}

// sum of the splits' partial rows in split order, times the head's gate
template <typename T>
__global__ void sigmoid_attn_merge_kernel(const float* __restrict__ partial, int splits, const T* __restrict__ gate, long gate_stride, T* __restrict__ out, long n_tokens, int H, int dv) {
    const long n = n_tokens * H * dv;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; k++) s += partial[k * n + i];
        const long th = i / dv, t = th / H;
        const int h = (int)(th - t * H);
        out[i] = from_f<T>(s * sigmoid_f(to_f(gate[t * gate_stride + h])));
    }
}

// ------------------------------------------------------------------------------------------------ gated linear attention
// grid (sequence portions, heads, column blocks of 32 value columns); 8 warps; thread (warp w, lane) keeps S[i][col] for a
// contiguous run of key channels i in registers.  Tokens run in order in chunks of kGlaChunk staged in shared memory; per token every
// warp leaves its part of o in shared memory, and the parts are summed in warp order once per chunk.  The arithmetic of a token
// does not depend on where a portion starts or ends.
constexpr int kGlaChunk = 16;
constexpr int kGlaWarps = 8;
constexpr int kGlaRows = 32;         // key channels per thread: dim <= 256
template <typename T, bool AHEAD>
__global__ void __launch_bounds__(256, AHEAD ? 2 : 3) gla_scan_kernel(const T* __restrict__ proj, long proj_stride, int q_off, int k_off, int v_off, const T* __restrict__ z, long z_stride,
                                                       const T* __restrict__ z_bias, float inv_tau, float q_scale, int H, int d, int dv, const int* __restrict__ seqs,
                                                       int seqs_stride, float* __restrict__ state, float* __restrict__ o_out) {
    extern __shared__ __align__(16) float sm[];
    // warp w owns the key channels w * rpt .. w * rpt + rpt - 1 (rpt a multiple of 4: float4 reads); channels >= d are zero
    const int rpt = (((d + kGlaWarps - 1) / kGlaWarps) + 3) & ~3, dp = rpt * kGlaWarps;
    float* qs = sm;                             // [chunk][dp]
    float* ks = qs + kGlaChunk * dp;            // [chunk][dp]
    float* as = ks + kGlaChunk * dp;            // [chunk][dp]
    float* vs = as + kGlaChunk * dp;            // [chunk][32]
    float* part = vs + kGlaChunk * 32;          // [chunk][warps][32]
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, col = c0 + lane;
    const int start = seqs[s], len = seqs[seqs_stride + s], rd = seqs[2 * seqs_stride + s], wr = seqs[3 * seqs_stride + s];
    const long srow = (long)H * d * dv;
    float S[kGlaRows];
#pragma unroll
    for (int r = 0; r < kGlaRows; r++) {
        const int i = warp * rpt + r;
        S[r] = (rd >= 0 && r < rpt && i < d && col < dv) ? state[rd * srow + ((long)h * d + i) * dv + col] : 0.f;
    }
    // the next chunk's inputs are fetched into registers while the current chunk runs, and turned into decays and staged afterwards
    constexpr int E = kGlaChunk * kGlaRows * kGlaWarps / 256;      // staged values per thread and array, at most
    float rq[E], rk[E], rz[E], rv[2];
    auto fetch = [&](int t0) {
        const int nt = min(kGlaChunk, len - t0);
#pragma unroll
        for (int e = 0; e < E; e++) {
            const int i = threadIdx.x + e * 256;
            rq[e] = rk[e] = rz[e] = 0.f;
            if (i < nt * dp) {
                const int tt = i / dp, c = i - tt * dp;
                const long row = (long)(start + t0 + tt);
                if (c < d) {
                    rq[e] = to_f(proj[row * proj_stride + q_off + h * d + c]);
                    rk[e] = to_f(proj[row * proj_stride + k_off + h * d + c]);
                    rz[e] = to_f(z[row * z_stride + h * d + c]) + to_f(z_bias[h * d + c]);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int i = threadIdx.x + e * 256, c = c0 + (i & 31);
            rv[e] = (i < nt * 32 && c < dv) ? to_f(proj[(long)(start + t0 + (i >> 5)) * proj_stride + v_off + h * dv + c]) : 0.f;
        }
    };
    if (AHEAD && len > 0) fetch(0);
    for (int t0 = 0; t0 < len; t0 += kGlaChunk) {
        const int nt = min(kGlaChunk, len - t0);
        if (!AHEAD) fetch(t0);      // decode steps: one token per sequence, nothing to run ahead of
        __syncthreads();
#pragma unroll
        for (int e = 0; e < E; e++) {
            const int i = threadIdx.x + e * 256;
            if (i < nt * dp) {
                const int c = i % dp;
                qs[i] = rq[e] * q_scale;
                ks[i] = rk[e];
                as[i] = c < d ? expf(log_sigmoid_f(rz[e]) * inv_tau) : 0.f;
            }
        }
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int i = threadIdx.x + e * 256;
            if (i < nt * 32) vs[i] = rv[e];
        }
        __syncthreads();
        if (AHEAD && t0 + kGlaChunk < len) fetch(t0 + kGlaChunk);
        for (int tt = 0; tt < nt; tt++) {
            const float v = vs[tt * 32 + lane];
            const float4* qr = reinterpret_cast<const float4*>(qs + tt * dp + warp * rpt);
            const float4* kr = reinterpret_cast<const float4*>(ks + tt * dp + warp * rpt);
            const float4* ar = reinterpret_cast<const float4*>(as + tt * dp + warp * rpt);
            float po = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < kGlaRows / 4; r4++) {
                if (4 * r4 < rpt) {
                    const float4 a = ar[r4], k = kr[r4], qv = qr[r4];
                    S[4 * r4] = fmaf(a.x, S[4 * r4], k.x * v);
                    po = fmaf(S[4 * r4], qv.x, po);
                    S[4 * r4 + 1] = fmaf(a.y, S[4 * r4 + 1], k.y * v);
                    po = fmaf(S[4 * r4 + 1], qv.y, po);
                    S[4 * r4 + 2] = fmaf(a.z, S[4 * r4 + 2], k.z * v);
                    po = fmaf(S[4 * r4 + 2], qv.z, po);
                    S[4 * r4 + 3] = fmaf(a.w, S[4 * r4 + 3], k.w * v);
                    po = fmaf(S[4 * r4 + 3], qv.w, po);
                }
            }
            part[(tt * kGlaWarps + warp) * 32 + lane] = po;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
            const int tt = i >> 5, c = c0 + (i & 31);
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < kGlaWarps; w++) o += part[(tt * kGlaWarps + w) * 32 + (i & 31)];
            if (c < dv) o_out[((long)(start + t0 + tt) * H + h) * dv + c] = o;
        }
    }
    if (wr >= 0) {
#pragma unroll
        for (int r = 0; r < kGlaRows; r++) {
            const int i = warp * rpt + r;
            if (r < rpt && i < d && col < dv) state[wr * srow + ((long)h * d + i) * dv + col] = S[r];
        }
    }
}

// out[t][h][c] = o[t][h][c] / sqrt(mean_c o^2 + eps) * w[c] * silu(gate[t][h][c]); a warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(256) gla_out_kernel(const float* __restrict__ o, const T* __restrict__ w, float eps, const T* __restrict__ gate, long gate_stride,
                                                      T* __restrict__ out, long n_rows, int H, int dv) {
    const int lane = threadIdx.x & 31;
    for (long row = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows; row += (long)gridDim.x * (blockDim.x >> 5)) {
        const float* src = o + row * dv;
        float s = 0.f;
        for (int c = lane; c < dv; c += 32) s += src[c] * src[c];
        s = warp_sum(s);
        const float inv = 1.0f / sqrtf(s / (float)dv + eps);
        const long t = row / H;
        const int h = (int)(row - t * H);
        for (int c = lane; c < dv; c += 32) out[row * dv + c] = from_f<T>(src[c] * inv * to_f(w[c]) * act_silu(to_f(gate[t * gate_stride + (long)h * dv + c])));
    }
}

// ------------------------------------------------------------------------------------------------ xIELU
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ z, T* __restrict__ out, const float* __restrict__ pq, long n) {
    const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float v = to_f(z[i]);
        out[i] = from_f<T>(v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v));
    }
}

// ------------------------------------------------------------------------------------------------ gated activation
// out[t][i] = gated_act(gate[t * stride + i], up[t * stride + i]) (seq_common.cuh); rows [gate F | up F]: up = gate + F, stride = 2 F
template <typename T>
__global__ void gated_act_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up, long stride, T* __restrict__ out, long n_rows, int F, int act, float limit) {
    const long n = n_rows * F;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const long t = i / F;
        const int c = (int)(i - t * F);
        out[i] = from_f<T>(gated_act(to_f(gate[t * stride + c]), to_f(up[t * stride + c]), act, limit));
    }
}
// out = relu(z)^2, element by element
template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ z, T* __restrict__ out, long n) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float r = fmaxf(to_f(z[i]), 0.f);
        out[i] = from_f<T>(r * r);
    }
}
// out = c tanh(z / c) in fp32, element by element
template <typename T>
__global__ void softcap_kernel(const T* __restrict__ z, float* __restrict__ out, long n, float cap) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = cap * tanhf(to_f(z[i]) / cap);
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

static int grid_for(long n, int per_block) {
    const long b = (n + per_block - 1) / per_block;
    return (int)(b < 148 * 8 ? (b < 1 ? 1 : b) : 148 * 8);
}

extern "C" int ktb200_group_rmsnorm_sandwich(const float* x_in, const void* y, int y_type, const void* w_post, const float* row_add, float* x_out, const void* w_pre,
                                             void* h_out, int groups, float eps, float weight_offset, int n_tokens, int width, int dtype, void* stream) {
    if (n_tokens <= 0) return KTB200_OK;
    if (!y || groups <= 0 || width <= 0 || width % groups || (w_pre && !h_out) || (!x_out && !h_out) || (y_type != KTB200_TYPE_BF16 && y_type != KTB200_TYPE_F32)) {
        set_error("group_rmsnorm_sandwich: bad argument");
        return KTB200_EINVAL;
    }
    const int stash = (size_t)width * sizeof(float) <= 160 * 1024 || !x_out;
    if (!stash && !x_out) { set_error("group_rmsnorm_sandwich: row too wide"); return KTB200_EINVAL; }
    const size_t smem = (32 + (stash ? (size_t)width : 0)) * sizeof(float);
    SEQ_DISPATCH(dtype, {
        GRANT_SMEM(sandwich_norm_kernel<T>, smem);
        sandwich_norm_kernel<T><<<n_tokens, 256, smem, (cudaStream_t)stream>>>(x_in, y, y_type, (const T*)w_post, row_add, x_out, (const T*)w_pre, (T*)h_out, groups, eps, width, stash, weight_offset);
    });
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_qk_norm_cache_write(const void* proj, long proj_stride, int heads, int kv_heads, int dim, int vdim, const void* q_norm_w, const void* k_norm_w, float eps,
                                          float temp_coef, int temp_every, const int* pos, const int* slot, const int* page_table, int max_pages, int page_size, void* cache,
                                          void* q_out, int n_tokens, int dtype, void* stream) {
    if (!proj || !q_norm_w || !k_norm_w || !pos || !slot || !page_table || !cache || !q_out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 ||
        temp_every <= 0 || page_size <= 0 || max_pages <= 0) {
        set_error("qk_norm_cache_write: bad argument");
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (qk_norm_cache_write_kernel<T><<<n_tokens, 256, 0, (cudaStream_t)stream>>>((const T*)proj, proj_stride, heads, kv_heads, dim, vdim, (const T*)q_norm_w,
                                                                                                   (const T*)k_norm_w, eps, temp_coef, temp_every, pos, slot, page_table,
                                                                                                   max_pages, page_size, (T*)cache, (T*)q_out)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" size_t ktb200_sigmoid_bias_attn_workspace(int n_tokens, int heads, int vdim, int splits) {
    return splits > 1 ? (size_t)splits * n_tokens * heads * vdim * sizeof(float) : 0;
}

extern "C" int ktb200_sigmoid_bias_attn_uses_tensor_cores(int heads, int kv_heads, int dim, int vdim, int dtype) {
    return dtype == KTB200_TYPE_BF16 && kv_heads > 0 && heads % kv_heads == 0 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 128 && vdim <= 128;
}
extern "C" int ktb200_sigmoid_bias_attn_tiles(int heads, int kv_heads, int n_tokens, int n_seqs) {
    return n_seqs + n_tokens / (kMmaRows / mma_heads_per_tile(heads / kv_heads));
}

extern "C" int ktb200_sigmoid_bias_attn(const void* q, int heads, int kv_heads, int dim, int vdim, float scale, const float* bias, int n_bias, const float* head_bias,
                                        const int* pos, const int* slot, const int* seqs, int seqs_stride, int n_seqs, const int* page_table, int max_pages, int page_size,
                                        const void* cache, const void* gate, long gate_stride, void* out, int n_tokens, int splits, float* workspace, int dtype,
                                        int allow_tensor_cores, void* stream) {
    if (!q || !bias || !head_bias || !pos || !slot || !page_table || !cache || !gate || !out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 ||
        vdim > 32 * kAttnMaxCols || n_bias <= 0 || splits < 1 || (splits > 1 && !workspace)) {
        set_error("sigmoid_bias_attn: bad argument");
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    if (allow_tensor_cores && seqs && n_seqs > 0 && ktb200_sigmoid_bias_attn_uses_tensor_cores(heads, kv_heads, dim, vdim, dtype)) {
        const int RH = mma_heads_per_tile(heads / kv_heads);
        const dim3 grid(ktb200_sigmoid_bias_attn_tiles(heads, kv_heads, n_tokens, n_seqs), kv_heads * (heads / kv_heads / RH), splits);
        // 64 rows x 32 keys per ring stage: 128 registers and ~52 KB, four CTAs (16 warps) per SM, for prompt portions and decode steps alike
        const size_t smem = (((size_t)kMmaRows + 2 * 32) * (dim + kMmaPad) + (size_t)2 * 32 * (vdim + kMmaPad)) * sizeof(__nv_bfloat16);
        using B = __nv_bfloat16;
#define MMA_LAUNCH(DK, DV)                                                                                                                                         \
    do {                                                                                                                                                           \
        GRANT_SMEM((sigmoid_attn_mma_kernel<DK, DV, kMmaRows, 32>), smem);                                                                                         \
        sigmoid_attn_mma_kernel<DK, DV, kMmaRows, 32><<<grid, kMmaRows * 2, smem, (cudaStream_t)stream>>>((const B*)q, heads, kv_heads, dim, vdim, scale, bias, n_bias,      \
                                                                                                          head_bias, pos, slot, seqs, seqs_stride, n_seqs, RH, page_table, \
                                                                                                          max_pages, page_size, (const B*)cache, (const B*)gate,           \
                                                                                                          gate_stride, (B*)out, splits > 1 ? workspace : nullptr, n_tokens); \
    } while (0)
        if (dim <= 64 && vdim <= 64) MMA_LAUNCH(4, 4);
        else MMA_LAUNCH(8, 8);
#undef MMA_LAUNCH
        KTB_LAUNCH_CHECK();
        if (splits > 1) {
            sigmoid_attn_merge_kernel<B><<<grid_for((long)n_tokens * heads * vdim, 256), 256, 0, (cudaStream_t)stream>>>(workspace, splits, (const B*)gate, gate_stride, (B*)out,
                                                                                                                       n_tokens, heads, vdim);
            KTB_LAUNCH_CHECK();
        }
        return KTB200_OK;
    }
    const int R = heads / kv_heads, HB = R < 8 ? R : 8, hblocks = (R + HB - 1) / HB;
    const size_t tiles = ((size_t)HB * dim + (size_t)kAttnTile * (dim + 1) + (size_t)kAttnTile * vdim) * sizeof(float);
    const int stage_bias = tiles + (size_t)HB * n_bias * sizeof(float) <= 96 * 1024;
    const size_t smem = tiles + (stage_bias ? (size_t)HB * n_bias * sizeof(float) : 0);
    if (smem > 200 * 1024) { set_error("sigmoid_bias_attn: head too wide for shared memory"); return KTB200_EINVAL; }
    SEQ_DISPATCH(dtype, {
        GRANT_SMEM(sigmoid_attn_kernel<T>, smem);
        sigmoid_attn_kernel<T><<<dim3(n_tokens, kv_heads * hblocks, splits), HB * 32, smem, (cudaStream_t)stream>>>(
            (const T*)q, heads, kv_heads, dim, vdim, scale, bias, n_bias, head_bias, pos, slot, page_table, max_pages, page_size, (const T*)cache, (const T*)gate, gate_stride,
            (T*)out, splits > 1 ? workspace : nullptr, n_tokens, stage_bias);
        KTB_LAUNCH_CHECK();
        if (splits > 1) {
            sigmoid_attn_merge_kernel<T><<<grid_for((long)n_tokens * heads * vdim, 256), 256, 0, (cudaStream_t)stream>>>(workspace, splits, (const T*)gate, gate_stride, (T*)out,
                                                                                                                       n_tokens, heads, vdim);
            KTB_LAUNCH_CHECK();
        }
    });
    return KTB200_OK;
}

extern "C" int ktb200_gla_scan(const void* proj, long proj_stride, int q_off, int k_off, int v_off, const void* z, long z_stride, const void* z_bias, float tau, int heads,
                               int dim, int vdim, const int* seqs, int seqs_stride, int n_seqs, int n_tokens, float* state, float* o_out, int dtype, void* stream) {
    if (!proj || !z || !z_bias || !seqs || !state || !o_out || heads <= 0 || dim <= 0 || dim > kGlaWarps * kGlaRows || vdim <= 0 || !(tau > 0.f)) {
        set_error("gla_scan: bad argument (dim <= %d)", kGlaWarps * kGlaRows);
        return KTB200_EINVAL;
    }
    if (n_seqs <= 0) return KTB200_OK;
    const int dp = ((((dim + kGlaWarps - 1) / kGlaWarps) + 3) & ~3) * kGlaWarps;      // key channels padded to whole float4 per warp
    const size_t smem = ((size_t)3 * kGlaChunk * dp + kGlaChunk * 32 + (size_t)kGlaChunk * kGlaWarps * 32) * sizeof(float);
#define GLA_LAUNCH(AHEAD)                                                                                                                                         \
    SEQ_DISPATCH(dtype, {                                                                                                                                         \
        GRANT_SMEM((gla_scan_kernel<T, AHEAD>), smem);                                                                                                            \
        gla_scan_kernel<T, AHEAD><<<dim3(n_seqs, heads, (vdim + 31) / 32), kGlaWarps * 32, smem, (cudaStream_t)stream>>>(                                         \
            (const T*)proj, proj_stride, q_off, k_off, v_off, (const T*)z, z_stride, (const T*)z_bias, 1.0f / tau, 1.0f / sqrtf((float)dim), heads, dim, vdim, seqs, \
            seqs_stride, state, o_out);                                                                                                                           \
    })
    if (n_tokens > n_seqs) GLA_LAUNCH(true);      // some portion has several tokens: fetch a chunk ahead
    else GLA_LAUNCH(false);
#undef GLA_LAUNCH
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_gla_out(const float* o, const void* norm_w, float eps, const void* gate, long gate_stride, void* out, int n_tokens, int heads, int vdim, int dtype,
                              void* stream) {
    if (!o || !norm_w || !gate || !out || heads <= 0 || vdim <= 0) { set_error("gla_out: bad argument"); return KTB200_EINVAL; }
    if (n_tokens <= 0) return KTB200_OK;
    const long rows = (long)n_tokens * heads;
    SEQ_DISPATCH(dtype, (gla_out_kernel<T><<<grid_for(rows, 8), 256, 0, (cudaStream_t)stream>>>(o, (const T*)norm_w, eps, (const T*)gate, gate_stride, (T*)out, rows, heads, vdim)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_xielu(const void* z, void* out, const float* pq, long n, int dtype, void* stream) {
    if (!z || !out || !pq) { set_error("xielu: bad argument"); return KTB200_EINVAL; }
    if (n <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (xielu_kernel<T><<<grid_for(n, 256 * 4), 256, 0, (cudaStream_t)stream>>>((const T*)z, (T*)out, pq, n)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_gated_act_mul(const void* gate, const void* up, long in_stride, void* out, int n_tokens, int ff, int act, float limit, int dtype, void* stream) {
    if (!gate || !up || !out || ff <= 0 || in_stride < ff || act < kActSilu || act > kActClampedGlu) { set_error("gated_act_mul: bad argument"); return KTB200_EINVAL; }
    if (n_tokens <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (gated_act_mul_kernel<T><<<grid_for((long)n_tokens * ff, 256 * 4), 256, 0, (cudaStream_t)stream>>>((const T*)gate, (const T*)up, in_stride, (T*)out,
                                                                                                                         n_tokens, ff, act, limit)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_relu_squared(const void* z, void* out, long n, int dtype, void* stream) {
    if (!z || !out) { set_error("relu_squared: bad argument"); return KTB200_EINVAL; }
    if (n <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (relu_squared_kernel<T><<<grid_for(n, 256 * 4), 256, 0, (cudaStream_t)stream>>>((const T*)z, (T*)out, n)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_softcap(const void* z, float* out, long n, float cap, int dtype, void* stream) {
    if (!z || !out || !(cap > 0.f)) { set_error("softcap: bad argument"); return KTB200_EINVAL; }
    if (n <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (softcap_kernel<T><<<grid_for(n, 256 * 4), 256, 0, (cudaStream_t)stream>>>((const T*)z, out, n, cap)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}
