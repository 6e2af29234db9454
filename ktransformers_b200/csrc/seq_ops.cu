// Token-major operators of decoder layers that keep a 32-bit residual stream and per-sequence state (libktb200_seq.so).
//
//   ktb200_group_rmsnorm_shift   x_out = x_in + mult * (a + b) + row   (each optional; row: one vector for all tokens), then RMS norm in `groups` equal parts, then an
//                                optional token shift  hs_t = h_t + (h_{t-1} - h_t) * mu  whose h_{t-1} comes from the same
//                                step (recomputed from the previous row) or from the per-sequence state rows
//   ktb200_latent_prep           what follows the fused down-projections of latent attention: RMS norm of the query latent,
//                                RMS norm of the key/value latent, rotation of the shared rotated key part, paged cache write
//   ktb200_sigmoid_gate_mul      heads [H][T][dv] * sigmoid(gate [T][H*dv]) -> [T][H*dv]
//   ktb200_poly_norm             a N(z) + b N(z^2) + c N(z^3) + e,  N(y) = y / sqrt(mean(y^2) + eps) over a token's row
//   ktb200_experts_gate_up/_down per (token, slot) pair GEMVs over dense (bf16 / f32) expert weights: a gated activation of (gate, up)
//                                (seq_common.cuh: SiLU, tanh-GELU or the clamped sigmoid form), then the weighted sum of the chosen
//                                experts' down projections in fp32
//
// Every kernel is templated on the storage type T (bf16 or float) of activations and weights; norms, angles, the residual
// sum, sigmoid / silu arguments and all reductions are fp32 (angles: fp64 tables).  Rows are addressed through per-token
// index arrays, so one launch serves a ragged batch of prompt portions and decode tokens alike.
#include <cuda_bf16.h>

#include "common.cuh"
#include "seq_common.cuh"

namespace ktb {

// ------------------------------------------------------------------------------------------------ norm + token shift
// One CTA per token.  smem: inv[2][groups] (padded to 16 bytes) | (stash) row[D] | prev row[D].  With `stash` the row (after the residual sum) and the
// previous token's row are read from global memory ONCE by all threads and kept in shared memory for the group sums and the
// output pass; rows too wide for shared memory are re-read instead.
constexpr int kNormBatch = 4;
template <typename T>
__global__ void __launch_bounds__(256) group_norm_shift_kernel(const float* __restrict__ x_in, const void* da, int a_type, const void* db, int b_type, float mult,
                                                               const float* __restrict__ row_add, float* __restrict__ x_out, const T* __restrict__ w, int groups, float eps, const T* __restrict__ mu,
                                                               const int* __restrict__ prev_idx, const int* __restrict__ rd_row, const int* __restrict__ wr_row,
                                                               float* __restrict__ state, T* __restrict__ h_out, T* __restrict__ hs_out, int D, int stash, int vec) {
    extern __shared__ __align__(16) float sm[];
    float* inv_cur = sm;
    float* inv_prev = sm + groups;
    float* cur = sm + ((2 * groups + 3) & ~3);      // 16-byte aligned: the staged rows are accessed as float4
    float* prv = cur + D;
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int gs = D / groups;
    const bool add = da != nullptr || db != nullptr || row_add != nullptr;
    const int pi = (mu && prev_idx) ? prev_idx[t] : -1;      // row of the previous token inside this step, or -1
    const int rr = (mu && rd_row) ? rd_row[t] : -1;
    const int wr = (mu && wr_row) ? wr_row[t] : -1;
    auto row_val = [&](int r, int i) -> float {
        float v = x_in[(long)r * D + i];
        if (add) {
            float s = 0.f;
            if (da) s += load_hidden(da, (long)r * D + i, a_type);
            if (db) s += load_hidden(db, (long)r * D + i, b_type);
            v = v + mult * s;
            if (row_add) v += row_add[i];
        }
        return v;
    };
    auto row_val4 = [&](int r, int i) -> float4 {
        float4 v = load4(x_in + (long)r * D + i);
        if (add) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            if (da) { const float4 u = load4_hidden(da, (long)r * D + i, a_type); s.x += u.x; s.y += u.y; s.z += u.z; s.w += u.w; }
            if (db) { const float4 u = load4_hidden(db, (long)r * D + i, b_type); s.x += u.x; s.y += u.y; s.z += u.z; s.w += u.w; }
            v.x = v.x + mult * s.x; v.y = v.y + mult * s.y; v.z = v.z + mult * s.z; v.w = v.w + mult * s.w;
            if (row_add) { const float4 u = load4(row_add + i); v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w; }
        }
        return v;
    };
    if (stash) {
        if (vec) {      // kNormBatch independent 16-byte loads per array in flight before the first use
            for (int base = 0; base < D; base += blockDim.x * 4 * kNormBatch) {
                float4 v[kNormBatch], u[kNormBatch];
#pragma unroll
                for (int k = 0; k < kNormBatch; k++) {
                    const int i = base + (k * blockDim.x + tid) * 4;
                    if (i < D) {
                        v[k] = row_val4(t, i);
                        if (pi >= 0) u[k] = row_val4(pi, i);
                    }
                }
#pragma unroll
                for (int k = 0; k < kNormBatch; k++) {
                    const int i = base + (k * blockDim.x + tid) * 4;
                    if (i < D) {
                        store4(cur + i, v[k]);
                        if (pi >= 0) store4(prv + i, u[k]);
                    }
                }
            }
        } else {
            for (int i = tid; i < D; i += blockDim.x) {
                cur[i] = row_val(t, i);
                if (pi >= 0) prv[i] = row_val(pi, i);
            }
        }
        __syncthreads();
    }
    if (stash && vec && nw % groups == 0 && gs % (4 * (nw / groups)) == 0) {
        // every warp sums one of nw equal chunks (a group = nw / groups consecutive chunks); partial sums meet in shared memory
        const int per = nw / groups, chunk = gs / per, g = warp / per;
        const float* c = cur + g * gs + (warp % per) * chunk;
        const float* q = prv + g * gs + (warp % per) * chunk;
        float sc = 0.f, sp = 0.f;
        for (int i = lane * 4; i < chunk; i += 128) {
            const float4 v = load4(c + i);
            sc += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            if (pi >= 0) {
                const float4 u = load4(q + i);
                sp += (u.x * u.x + u.y * u.y) + (u.z * u.z + u.w * u.w);
            }
        }
        sc = warp_sum(sc);
        sp = warp_sum(sp);
        float* part = prv + D;                     // [2][nw] behind the staged rows
        if (lane == 0) { part[warp] = sc; part[nw + warp] = sp; }
        __syncthreads();
        if (warp == 0 && lane < groups) {
            float a = 0.f, b = 0.f;
            for (int k = 0; k < per; k++) { a += part[lane * per + k]; b += part[nw + lane * per + k]; }
            inv_cur[lane] = 1.0f / sqrtf(a / (float)gs + eps);
            inv_prev[lane] = 1.0f / sqrtf(b / (float)gs + eps);
        }
    } else
    for (int g = warp; g < groups; g += nw) {
        float sc = 0.f, sp = 0.f;
        for (int i = lane; i < gs; i += 32) {
            const float v = stash ? cur[g * gs + i] : row_val(t, g * gs + i);
            sc += v * v;
            if (pi >= 0) {
                const float u = stash ? prv[g * gs + i] : row_val(pi, g * gs + i);
                sp += u * u;
            }
        }
        sc = warp_sum(sc);
        sp = warp_sum(sp);
        if (lane == 0) {
            inv_cur[g] = 1.0f / sqrtf(sc / (float)gs + eps);
            inv_prev[g] = 1.0f / sqrtf(sp / (float)gs + eps);
        }
    }
    __syncthreads();
    if (vec && stash) {     // four columns per thread and pass: one group, 16- / 8-byte loads and stores, loads batched
        for (int base = 0; base < D; base += blockDim.x * 4 * kNormBatch) {
            float4 wv[kNormBatch], mv[kNormBatch], sv[kNormBatch];
#pragma unroll
            for (int k = 0; k < kNormBatch; k++) {
                const int i = base + (k * blockDim.x + tid) * 4;
                if (i < D) {
                    wv[k] = load4(w + i);
                    if (mu) mv[k] = load4(mu + i);
                    if (mu && pi < 0 && rr >= 0) sv[k] = load4(state + (long)rr * D + i);
                }
            }
#pragma unroll
            for (int k = 0; k < kNormBatch; k++) {
                const int i = base + (k * blockDim.x + tid) * 4;
                if (i >= D) continue;
                const float4 v = load4(cur + i);
                if (add && x_out) store4(x_out + (long)t * D + i, v);
                const float4 wi = wv[k];
                const float ic = inv_cur[i / gs];
                const float4 h = make_float4(v.x * ic * wi.x, v.y * ic * wi.y, v.z * ic * wi.z, v.w * ic * wi.w);
                if (h_out) store4(h_out + (long)t * D + i, h);
                if (mu) {
                    float4 hp = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (pi >= 0) {
                        const float4 u = load4(prv + i);
                        const float ip = inv_prev[i / gs];
                        hp = make_float4(u.x * ip * wi.x, u.y * ip * wi.y, u.z * ip * wi.z, u.w * ip * wi.w);
                    } else if (rr >= 0) {
                        hp = sv[k];
                    }
                    const float4 m4 = mv[k];
                    if (hs_out) store4(hs_out + (long)t * D + i, make_float4(h.x + (hp.x - h.x) * m4.x, h.y + (hp.y - h.y) * m4.y, h.z + (hp.z - h.z) * m4.z, h.w + (hp.w - h.w) * m4.w));
                    if (wr >= 0) store4(state + (long)wr * D + i, h);
                }
            }
        }
        return;
    }
    for (int i = tid; i < D; i += blockDim.x) {
        const float v = stash ? cur[i] : row_val(t, i);
        if (add && x_out) x_out[(long)t * D + i] = v;
        const float wi = to_f(w[i]);
        const float h = v * inv_cur[i / gs] * wi;
        if (h_out) h_out[(long)t * D + i] = from_f<T>(h);
        if (mu) {
            float hp = 0.f;
            if (pi >= 0) hp = (stash ? prv[i] : row_val(pi, i)) * inv_prev[i / gs] * wi;
            else if (rr >= 0) hp = state[(long)rr * D + i];
            if (hs_out) hs_out[(long)t * D + i] = from_f<T>(h + (hp - h) * to_f(mu[i]));
            if (wr >= 0) state[(long)wr * D + i] = h;
        }
    }
}

// ------------------------------------------------------------------------------------------------ latent prep
// One CTA per token.  proj row = [ q latent (q_rank) | kv latent (kv_rank) | rotated key part (rot_dim) | ... ].
template <typename T>
__global__ void __launch_bounds__(256) latent_prep_kernel(const T* __restrict__ proj, long proj_stride, int q_rank, int kv_rank, int rot_dim, int rot_dims, int rot_layout,
                                                          const double* __restrict__ inv_freq, const T* __restrict__ qn_w, const T* __restrict__ kvn_w, float eps,
                                                          const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ page_table, int max_pages,
                                                          int page_size, T* __restrict__ cache, T* __restrict__ cq_out) {
    __shared__ float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const T* p = proj + (long)t * proj_stride;
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < q_rank; i += blockDim.x) { const float v = to_f(p[i]); sq += v * v; }
    for (int i = tid; i < kv_rank; i += blockDim.x) { const float v = to_f(p[q_rank + i]); sk += v * v; }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float iq = q_rank ? 1.0f / sqrtf(sq / (float)q_rank + eps) : 0.f;
    const float ik = 1.0f / sqrtf(sk / (float)kv_rank + eps);
    for (int i = tid; i < q_rank; i += blockDim.x) cq_out[(long)t * q_rank + i] = from_f<T>(to_f(p[i]) * iq * to_f(qn_w[i]));
    const int ps = pos[t];
    const long row = (long)page_table[(long)slot[t] * max_pages + (ps / page_size) % max_pages] * page_size + ps % page_size;
    T* c = cache + row * (kv_rank + rot_dim);
    for (int i = tid; i < kv_rank; i += blockDim.x) c[i] = from_f<T>(to_f(p[q_rank + i]) * ik * to_f(kvn_w[i]));
    const T* kr = p + q_rank + kv_rank;
    for (int i = tid; i < rot_dim; i += blockDim.x) {
        float v = to_f(kr[i]);
        if (i < rot_dims) v = rot_turn(v, to_f(kr[rot_partner(i, rot_dims, rot_layout)]), i, rot_dims, rot_layout, ps, inv_freq);
        c[kv_rank + i] = from_f<T>(v);
    }
}

// ------------------------------------------------------------------------------------------------ rotated query part
// out[t][h][:] = rot(q[t][h][dn : dn + dr]) at position pos[t] (pairs of either layout over the first rot_dims columns)
template <typename T>
__global__ void rope_rows_kernel(const T* __restrict__ q, int H, int dn, int dr, int rot_dims, int rot_layout, const double* __restrict__ inv_freq, const int* __restrict__ pos,
                                 T* __restrict__ out, int n_tokens) {
    const long n = (long)n_tokens * H * dr;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const int d = (int)(i % dr);
        const long th = i / dr;
        const T* src = q + th * (dn + dr) + dn;
        float v = to_f(src[d]);
        if (d < rot_dims) v = rot_turn(v, to_f(src[rot_partner(d, rot_dims, rot_layout)]), d, rot_dims, rot_layout, pos[th / H], inv_freq);
        out[i] = from_f<T>(v);
    }
}

// ------------------------------------------------------------------------------------------------ output gate
template <typename T>
__global__ void sigmoid_gate_mul_kernel(const T* __restrict__ heads, const T* __restrict__ gate, long gate_stride, T* __restrict__ out, int n_tokens, int H, int dv) {
    const long n = (long)n_tokens * H * dv;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const int d = (int)(i % dv);
        const int h = (int)((i / dv) % H);
        const long t = i / ((long)dv * H);
        const float o = to_f(heads[((long)h * n_tokens + t) * dv + d]);
        const float g = to_f(gate[t * gate_stride + (long)h * dv + d]);
        out[i] = from_f<T>(o * (1.0f / (1.0f + expf(-g))));
    }
}

// ------------------------------------------------------------------------------------------------ PolyNorm
template <typename T>
__global__ void __launch_bounds__(256) poly_norm_kernel(const T* __restrict__ z, T* __restrict__ out, const float* __restrict__ coef, float eps, int F) {
    __shared__ float red[32];
    const long t = blockIdx.x;
    const T* zr = z + t * F;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = to_f(zr[i]), v2 = v * v, v3 = v2 * v;
        s1 += v2; s2 += v2 * v2; s3 += v3 * v3;
    }
    s1 = block_sum(s1, red); s2 = block_sum(s2, red); s3 = block_sum(s3, red);
    const float a = coef[0] / sqrtf(s1 / (float)F + eps), b = coef[1] / sqrtf(s2 / (float)F + eps), c = coef[2] / sqrtf(s3 / (float)F + eps), e = coef[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = to_f(zr[i]);
        out[t * F + i] = from_f<T>(a * v + b * v * v + c * v * v * v + e);
    }
}

// ------------------------------------------------------------------------------------------------ dense experts, per pair
// Two kinds of expert: gated (gated_act(W_gate x, W_up x), seq_common.cuh) and, with no gate matrix (Wg == nullptr), relu(W_up x)^2.
__device__ __forceinline__ float act_relu_sq(float x) { const float r = fmaxf(x, 0.f); return r * r; }
// grid (pairs, row blocks); a warp owns ff rows r = blockIdx.y * nw + warp (+ stride); the token's row sits in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) experts_gate_up_kernel(const T* __restrict__ x, const int64_t* __restrict__ ids, int top, const T* __restrict__ Wg, const T* __restrict__ Wu,
                                                              T* __restrict__ act, int D, int F, int act_kind, float limit) {
    extern __shared__ __align__(16) float xs[];
    const long p = blockIdx.x;
    const long t = p / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int i = threadIdx.x; i < D; i += blockDim.x) xs[i] = to_f(x[t * D + i]);
    __syncthreads();
    const long e = ids[p];
    const T* u = Wu + e * (long)F * D;
    if (!Wg) {      // experts without a gate matrix: relu(up)^2
        const bool vec = rows_vectorise(Wu, D);
        for (int r = blockIdx.y * nw + warp; r < F; r += gridDim.y * nw) {
            const float su = warp_sum(lane_dot(u + (long)r * D, xs, D, lane, vec));
            if (lane == 0) act[p * F + r] = from_f<T>(act_relu_sq(su));
        }
        return;
    }
    const T* g = Wg + e * (long)F * D;
    const bool vec = rows_vectorise(Wg, D) && rows_vectorise(Wu, D);
    for (int r = blockIdx.y * nw + warp; r < F; r += gridDim.y * nw) {
        float sg = lane_dot(g + (long)r * D, xs, D, lane, vec);
        float su = lane_dot(u + (long)r * D, xs, D, lane, vec);
        sg = warp_sum(sg);
        su = warp_sum(su);
        if (lane == 0) act[p * F + r] = from_f<T>(gated_act(sg, su, act_kind, limit));
    }
}

// grid (tokens, row blocks); out[t][d] = sum_j w[t][j] * Wd[ids[t][j]][d] . act[t*top + j]   (fp32, slot order)
template <typename T>
__global__ void __launch_bounds__(256) experts_down_kernel(const T* __restrict__ act, const int64_t* __restrict__ ids, const float* __restrict__ wts, int top,
                                                           const T* __restrict__ Wd, float* __restrict__ out, int D, int F) {
    extern __shared__ __align__(16) float as[];   // [top][F]
    const long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int i = threadIdx.x; i < top * F; i += blockDim.x) as[i] = to_f(act[t * top * F + i]);
    __syncthreads();
    const bool vec = rows_vectorise(Wd, F);
    for (int d = blockIdx.y * nw + warp; d < D; d += gridDim.y * nw) {
        float acc = 0.f;      // this lane's share of sum_j w_j * (row . act_j): ONE warp reduction per output row, and the
        for (int j = 0; j < top; j++) {   // next expert's loads are not held up behind a shuffle chain
            const T* wd = Wd + (ids[t * top + j] * (long)D + d) * F;
            acc = fmaf(wts[t * top + j], lane_dot(wd, as + j * F, F, lane, vec), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) out[t * D + d] = acc;
    }
}

// ------------------------------------------------------------------------------------------------ dense experts, by expert
// Batches of a few tokens: grid (experts, row blocks).  A CTA lists the pairs routed to ITS expert from the id array (in pair
// order, so the result does not depend on the schedule), stages the rows of up to NT (2 or 4) of them in shared memory in
// the operand type, and applies every weight row it streams to all of them: an expert's weights cross HBM once per
// NT pairs instead of once per pair.  Per pair the products are summed in the order of the per-pair kernels.

// pairs p (ascending) with ids[p] == e into list[0..n), n into list[P]; all threads of the CTA call it
__device__ __forceinline__ int list_pairs_of_expert(const int64_t* __restrict__ ids, int P, int e, int* list) {
    const int lane = threadIdx.x & 31;
    if (threadIdx.x < 32) {
        int n = 0;
        for (int base = 0; base < P; base += 32) {
            const int p = base + lane;
            const bool hit = p < P && ids[p] == e;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            if (hit) list[n + __popc(m & ((1u << lane) - 1u))] = p;
            n += __popc(m);
        }
        if (lane == 0) list[P] = n;
    }
    __syncthreads();
    return list[P];
}

template <typename T> __device__ __forceinline__ void stage_rows(T* dst, const T* __restrict__ src, const int* rows, int div, int m, int n, bool vec) {
    for (int k = 0; k < m; k++) {
        const T* s = src + (long)(rows[k] / div) * n;
        if (vec) {
            constexpr int per = 16 / sizeof(T);
            for (int i = threadIdx.x * per; i < n; i += blockDim.x * per) *reinterpret_cast<uint4*>(dst + (long)k * n + i) = *reinterpret_cast<const uint4*>(s + i);
        } else {
            for (int i = threadIdx.x; i < n; i += blockDim.x) dst[(long)k * n + i] = s[i];
        }
    }
}

// s[q][k] += w[q] . xs[k] for k < m, this lane's share: NW weight rows against the same staged rows (each staged value is
// read from shared memory once for all of them, and NW 16-byte loads are in flight per lane)
template <int NT, int NW>
__device__ __forceinline__ void lane_dot_rows(const __nv_bfloat16* const (&w)[NW], const __nv_bfloat16* xs, int n, int m, int lane, bool vec, float (&s)[NW][NT]) {
    if (vec) {
        for (int i = lane * 8; i < n; i += 256) {
            uint4 v[NW];
#pragma unroll
            for (int q = 0; q < NW; q++) v[q] = ldg_stream16(w[q] + i);
#pragma unroll
            for (int k = 0; k < NT; k++) {
                if (k < m) {
                    const uint4 a = *reinterpret_cast<const uint4*>(xs + (long)k * n + i);
                    const float a0 = __uint_as_float(a.x << 16), a1 = __uint_as_float(a.x & 0xffff0000u), a2 = __uint_as_float(a.y << 16), a3 = __uint_as_float(a.y & 0xffff0000u);
                    const float a4 = __uint_as_float(a.z << 16), a5 = __uint_as_float(a.z & 0xffff0000u), a6 = __uint_as_float(a.w << 16), a7 = __uint_as_float(a.w & 0xffff0000u);
#pragma unroll
                    for (int q = 0; q < NW; q++) {
                        float t = s[q][k];
                        t = fmaf(__uint_as_float(v[q].x << 16), a0, t);
                        t = fmaf(__uint_as_float(v[q].x & 0xffff0000u), a1, t);
                        t = fmaf(__uint_as_float(v[q].y << 16), a2, t);
                        t = fmaf(__uint_as_float(v[q].y & 0xffff0000u), a3, t);
                        t = fmaf(__uint_as_float(v[q].z << 16), a4, t);
                        t = fmaf(__uint_as_float(v[q].z & 0xffff0000u), a5, t);
                        t = fmaf(__uint_as_float(v[q].w << 16), a6, t);
                        t = fmaf(__uint_as_float(v[q].w & 0xffff0000u), a7, t);
                        s[q][k] = t;
                    }
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            float wv[NW];
#pragma unroll
            for (int q = 0; q < NW; q++) wv[q] = __bfloat162float(w[q][i]);
#pragma unroll
            for (int k = 0; k < NT; k++) {
                if (k < m) {
                    const float xv = __bfloat162float(xs[(long)k * n + i]);
#pragma unroll
                    for (int q = 0; q < NW; q++) s[q][k] = fmaf(wv[q], xv, s[q][k]);
                }
            }
        }
    }
}
template <int NT, int NW>
__device__ __forceinline__ void lane_dot_rows(const float* const (&w)[NW], const float* xs, int n, int m, int lane, bool vec, float (&s)[NW][NT]) {
    if (vec) {
        for (int i = lane * 4; i < n; i += 128) {
            uint4 v[NW];
#pragma unroll
            for (int q = 0; q < NW; q++) v[q] = ldg_stream16(w[q] + i);
#pragma unroll
            for (int k = 0; k < NT; k++) {
                if (k < m) {
                    const float4 a = *reinterpret_cast<const float4*>(xs + (long)k * n + i);
#pragma unroll
                    for (int q = 0; q < NW; q++) {
                        float t = s[q][k];
                        t = fmaf(__uint_as_float(v[q].x), a.x, t);
                        t = fmaf(__uint_as_float(v[q].y), a.y, t);
                        t = fmaf(__uint_as_float(v[q].z), a.z, t);
                        t = fmaf(__uint_as_float(v[q].w), a.w, t);
                        s[q][k] = t;
                    }
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            float wv[NW];
#pragma unroll
            for (int q = 0; q < NW; q++) wv[q] = w[q][i];
#pragma unroll
            for (int k = 0; k < NT; k++) {
                if (k < m) {
                    const float xv = xs[(long)k * n + i];
#pragma unroll
                    for (int q = 0; q < NW; q++) s[q][k] = fmaf(wv[q], xv, s[q][k]);
                }
            }
        }
    }
}

// shared memory: list[P + 1] ints (padded to 16 bytes) | rows [NT][D] of T.  A warp takes two ff rows at a time (gate and up of each).
template <typename T, int NT>
__global__ void __launch_bounds__(256) experts_gate_up_by_expert_kernel(const T* __restrict__ x, const int64_t* __restrict__ ids, int top, int P, const T* __restrict__ Wg,
                                                                        const T* __restrict__ Wu, T* __restrict__ act, int D, int F, int act_kind, float limit) {
    extern __shared__ __align__(16) unsigned char sm_raw[];
    int* list = reinterpret_cast<int*>(sm_raw);
    T* xs = reinterpret_cast<T*>(sm_raw + (((size_t)(P + 1) * sizeof(int) + 15) & ~(size_t)15));
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int n = list_pairs_of_expert(ids, P, e, list);
    if (n == 0) return;
    const T* g = Wg + (long)e * F * D;
    const T* u = Wu + (long)e * F * D;
    const bool vec = (!Wg || rows_vectorise(Wg, D)) && rows_vectorise(Wu, D) && rows_vectorise(x, D);
    for (int c = 0; c < n; c += NT) {
        const int m = n - c < NT ? n - c : NT;
        if (c) __syncthreads();      // the rows of the previous pairs are consumed
        stage_rows(xs, x, list + c, top, m, D, vec);
        __syncthreads();
        if (!Wg) {      // no gate matrix: four up rows at a time, relu(.)^2
            for (int r = (blockIdx.y * nw + warp) * 4; r < F; r += gridDim.y * nw * 4) {
                const T* const w[4] = {u + (long)r * D, u + (long)(r + 1 < F ? r + 1 : r) * D, u + (long)(r + 2 < F ? r + 2 : r) * D, u + (long)(r + 3 < F ? r + 3 : r) * D};
                float s[4][NT];
#pragma unroll
                for (int q = 0; q < 4; q++)
#pragma unroll
                    for (int k = 0; k < NT; k++) s[q][k] = 0.f;
                lane_dot_rows<NT, 4>(w, xs, D, m, lane, vec, s);
#pragma unroll
                for (int k = 0; k < NT; k++) {
                    if (k < m) {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const float a = warp_sum(s[q][k]);
                            if (lane == q && r + q < F) act[(long)list[c + k] * F + r + q] = from_f<T>(act_relu_sq(a));
                        }
                    }
                }
            }
            continue;
        }
        for (int r = (blockIdx.y * nw + warp) * 2; r < F; r += gridDim.y * nw * 2) {
            const int r1 = r + 1 < F ? r + 1 : r;      // an odd last row is done twice and stored once
            const T* const w[4] = {g + (long)r * D, u + (long)r * D, g + (long)r1 * D, u + (long)r1 * D};
            float s[4][NT];
#pragma unroll
            for (int q = 0; q < 4; q++)
#pragma unroll
                for (int k = 0; k < NT; k++) s[q][k] = 0.f;
            lane_dot_rows<NT, 4>(w, xs, D, m, lane, vec, s);
#pragma unroll
            for (int k = 0; k < NT; k++) {
                if (k < m) {
                    const float a0 = warp_sum(s[0][k]), b0 = warp_sum(s[1][k]), a1 = warp_sum(s[2][k]), b1 = warp_sum(s[3][k]);
                    if (lane == 0) {
                        T* o = act + (long)list[c + k] * F;
                        o[r] = from_f<T>(gated_act(a0, b0, act_kind, limit));
                        if (r1 != r) o[r1] = from_f<T>(gated_act(a1, b1, act_kind, limit));
                    }
                }
            }
        }
    }
}

// y[p][d] = Wd[ids[p]][d] . act[p]  (fp32, one row per pair); shared memory: list | rows [NT][F] of T.  A warp takes four rows at a time.
template <typename T, int NT>
__global__ void __launch_bounds__(256) experts_down_by_expert_kernel(const T* __restrict__ act, const int64_t* __restrict__ ids, int P, const T* __restrict__ Wd,
                                                                     float* __restrict__ y, int D, int F) {
    extern __shared__ __align__(16) unsigned char sm_raw[];
    int* list = reinterpret_cast<int*>(sm_raw);
    T* as = reinterpret_cast<T*>(sm_raw + (((size_t)(P + 1) * sizeof(int) + 15) & ~(size_t)15));
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int n = list_pairs_of_expert(ids, P, e, list);
    if (n == 0) return;
    const T* wd = Wd + (long)e * D * F;
    const bool vec = rows_vectorise(Wd, F) && rows_vectorise(act, F);
    for (int c = 0; c < n; c += NT) {
        const int m = n - c < NT ? n - c : NT;
        if (c) __syncthreads();
        stage_rows(as, act, list + c, 1, m, F, vec);
        __syncthreads();
        for (int d = (blockIdx.y * nw + warp) * 4; d < D; d += gridDim.y * nw * 4) {
            const T* w[4];
#pragma unroll
            for (int q = 0; q < 4; q++) w[q] = wd + (long)(d + q < D ? d + q : d) * F;
            const T* const wc[4] = {w[0], w[1], w[2], w[3]};
            float s[4][NT];
#pragma unroll
            for (int q = 0; q < 4; q++)
#pragma unroll
                for (int k = 0; k < NT; k++) s[q][k] = 0.f;
            lane_dot_rows<NT, 4>(wc, as, F, m, lane, vec, s);
#pragma unroll
            for (int k = 0; k < NT; k++) {
                if (k < m) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const float a = warp_sum(s[q][k]);
                        if (lane == q && d + q < D) y[(long)list[c + k] * D + d + q] = a;
                    }
                }
            }
        }
    }
}

// out[t][d] = sum_j w[t][j] * y[t * top + j][d], fp32, slot order
__global__ void __launch_bounds__(256) experts_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts, int top, float* __restrict__ out, long n, int D) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const long t = i / D;
        const int d = (int)(i - t * D);
        float acc = 0.f;
        for (int j = 0; j < top; j++) acc = fmaf(wts[t * top + j], y[(t * top + j) * D + d], acc);
        out[i] = acc;
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

extern "C" int ktb200_group_rmsnorm_shift(const float* x_in, const void* delta_a, int a_type, const void* delta_b, int b_type, float mult, const float* row_add, float* x_out,
                                          const void* weight, int groups, float eps, const void* shift, const int* prev_idx, const int* rd_row, const int* wr_row,
                                          float* state, void* h_out, void* hs_out, int n_tokens, int width, int dtype, void* stream) {
    if (!x_in || !weight || groups <= 0 || width <= 0 || width % groups || n_tokens < 0) { set_error("group_rmsnorm_shift: bad argument"); return KTB200_EINVAL; }
    if ((delta_a || delta_b || row_add) && (!x_out || x_out == x_in)) { set_error("group_rmsnorm_shift: the sum needs a separate output row buffer"); return KTB200_EINVAL; }
    if (shift && (!prev_idx || !rd_row || !wr_row || !state || !hs_out)) { set_error("group_rmsnorm_shift: shift needs its index rows, state and output"); return KTB200_EINVAL; }
    if (n_tokens == 0) return KTB200_OK;
    size_t smem = (size_t)((2 * groups + 3) & ~3) * sizeof(float);
    const int stash = smem + (2 * (size_t)width + 64) * sizeof(float) <= 160 * 1024;
    if (stash) smem += (2 * (size_t)width + 64) * sizeof(float);      // two staged rows + the warps' partial sums
    auto al = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    const int vec = width % 4 == 0 && (width / groups) % 4 == 0 && al(x_in, 16) && al(x_out, 16) && al(delta_a, 16) && al(delta_b, 16) && al(row_add, 16) && al(weight, 16) && al(shift, 16) &&
                    al(state, 16) && al(h_out, 16) && al(hs_out, 16);
    SEQ_DISPATCH(dtype, {
        static size_t granted = 48 * 1024;      // opt-in shared memory, raised once per size
        if (smem > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(group_norm_shift_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); granted = smem; }
        group_norm_shift_kernel<T><<<n_tokens, 256, smem, (cudaStream_t)stream>>>(x_in, delta_a, a_type, delta_b, b_type, mult, row_add, x_out, (const T*)weight, groups, eps,
                                                                                  (const T*)shift, prev_idx, rd_row, wr_row, state, (T*)h_out, (T*)hs_out, width, stash, vec);
    });
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_latent_prep(const void* proj, long proj_stride, int q_rank, int kv_rank, int rot_dim, int rot_dims, int rot_layout, const double* inv_freq, const void* q_norm_w,
                                  const void* kv_norm_w, float eps, const int* pos, const int* slot, const int* page_table, int max_pages, int page_size, void* cache,
                                  void* cq_out, int n_tokens, int dtype, void* stream) {
    if (!proj || !kv_norm_w || !pos || !slot || !page_table || !cache || kv_rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || q_rank < 0 ||
        (rot_layout != kRotInterleaved && rot_layout != kRotHalves) ||
        (q_rank && (!q_norm_w || !cq_out)) || (rot_dims && !inv_freq) || page_size <= 0 || max_pages <= 0) {
        set_error("latent_prep: bad argument");
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (latent_prep_kernel<T><<<n_tokens, 256, 0, (cudaStream_t)stream>>>((const T*)proj, proj_stride, q_rank, kv_rank, rot_dim, rot_dims, rot_layout, inv_freq, (const T*)q_norm_w,
                                                                                           (const T*)kv_norm_w, eps, pos, slot, page_table, max_pages, page_size, (T*)cache, (T*)cq_out)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_rope_rows(const void* q, int num_heads, int dim, int rot_dim, int rot_dims, int rot_layout, const double* inv_freq, const int* pos, void* out, int n_tokens, int dtype,
                                void* stream) {
    if (!q || !pos || !out || num_heads <= 0 || dim < 0 || rot_dim <= 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || (rot_dims && !inv_freq) ||
        (rot_layout != kRotInterleaved && rot_layout != kRotHalves)) {
        set_error("rope_rows: bad argument");
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    const long n = (long)n_tokens * num_heads * rot_dim;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    SEQ_DISPATCH(dtype, (rope_rows_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)q, num_heads, dim, rot_dim, rot_dims, rot_layout, inv_freq, pos, (T*)out, n_tokens)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_sigmoid_gate_mul(const void* heads, const void* gate, long gate_stride, void* out, int n_tokens, int num_heads, int vdim, int dtype, void* stream) {
    if (!heads || !gate || !out || num_heads <= 0 || vdim <= 0) { set_error("sigmoid_gate_mul: bad argument"); return KTB200_EINVAL; }
    if (n_tokens <= 0) return KTB200_OK;
    const long n = (long)n_tokens * num_heads * vdim;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    SEQ_DISPATCH(dtype, (sigmoid_gate_mul_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)heads, (const T*)gate, gate_stride, (T*)out, n_tokens, num_heads, vdim)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_poly_norm(const void* z, void* out, const float* coef, float eps, int n_tokens, int ff, int dtype, void* stream) {
    if (!z || !out || !coef || ff <= 0) { set_error("poly_norm: bad argument"); return KTB200_EINVAL; }
    if (n_tokens <= 0) return KTB200_OK;
    SEQ_DISPATCH(dtype, (poly_norm_kernel<T><<<n_tokens, 256, 0, (cudaStream_t)stream>>>((const T*)z, (T*)out, coef, eps, ff)));
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_experts_gate_up(const void* x, const int64_t* ids, int top, const void* w_gate, const void* w_up, void* act, int n_tokens, int width, int ff, int act_kind,
                                      float limit, int dtype, void* stream) {
    if (!x || !ids || !w_up || !act || top <= 0 || width <= 0 || ff <= 0 || width * sizeof(float) > 200 * 1024 || act_kind < kActSilu || act_kind > kActClampedGlu) { set_error("experts_gate_up: bad argument"); return KTB200_EINVAL; }
    if (n_tokens <= 0) return KTB200_OK;
    const size_t smem = (size_t)width * sizeof(float);
    int ry = (ff + 7) / 8;   // row blocks: enough CTAs to fill 148 SMs several times over when there are few pairs
    { const int want = (148 * 8 + n_tokens * top - 1) / (n_tokens * top); if (ry > want) ry = want; if (ry < 1) ry = 1; }
    SEQ_DISPATCH(dtype, {
        static size_t granted = 48 * 1024;
        if (smem > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(experts_gate_up_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); granted = smem; }
        experts_gate_up_kernel<T><<<dim3(n_tokens * top, ry), 256, smem, (cudaStream_t)stream>>>((const T*)x, ids, top, (const T*)w_gate, (const T*)w_up, (T*)act, width, ff, act_kind, limit);
    });
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_experts_down(const void* act, const int64_t* ids, const float* weights, int top, const void* w_down, float* out, int n_tokens, int width, int ff, int dtype,
                                   void* stream) {
    if (!act || !ids || !weights || !w_down || !out || top <= 0 || width <= 0 || ff <= 0 || (size_t)top * ff * sizeof(float) > 200 * 1024) { set_error("experts_down: bad argument"); return KTB200_EINVAL; }
    if (n_tokens <= 0) return KTB200_OK;
    const size_t smem = (size_t)top * ff * sizeof(float);
    int ry = (width + 7) / 8;
    { const int want = (148 * 8 + n_tokens - 1) / n_tokens; if (ry > want) ry = want; if (ry < 1) ry = 1; }
    SEQ_DISPATCH(dtype, {
        static size_t granted = 48 * 1024;
        if (smem > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(experts_down_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); granted = smem; }
        experts_down_kernel<T><<<dim3(n_tokens, ry), 256, smem, (cudaStream_t)stream>>>((const T*)act, ids, weights, top, (const T*)w_down, out, width, ff);
    });
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

static size_t by_expert_smem(int pairs, int staged, size_t row_bytes) { return (((size_t)(pairs + 1) * sizeof(int) + 15) & ~(size_t)15) + staged * row_bytes; }
static int by_expert_row_blocks(int rows, int rows_per_warp, int pairs, int n_experts) {      // enough CTAs to fill 148 SMs several times over with the experts that can be active
    const int active = pairs < n_experts ? pairs : n_experts;
    int ry = (rows + 8 * rows_per_warp - 1) / (8 * rows_per_warp);
    const int want = (148 * 8 + active - 1) / active;
    if (ry > want) ry = want;
    return ry < 1 ? 1 : ry;
}
// pairs staged per pass: 4 once there are as many pairs as experts (several pairs per expert become likely), else 2 (smaller CTAs, more of them per SM)
static int by_expert_staged(int staged, int pairs, int n_experts) { return staged == 2 || staged == 4 ? staged : (pairs >= n_experts ? 4 : 2); }

#define BY_EXPERT_LAUNCH(kernel, rows, rows_per_warp, row_bytes, ...)                                                                                     \
    SEQ_DISPATCH(dtype, {                                                                                                                                  \
        const size_t smem = by_expert_smem(P, NT, (row_bytes) * sizeof(T));                                                                                \
        if (smem > 200 * 1024) { set_error(#kernel ": rows too long for shared memory"); return KTB200_EINVAL; }                                           \
        static size_t granted = 48 * 1024;                                                                                                                 \
        if (smem > granted) { KTB_CUDA_CHECK(cudaFuncSetAttribute(kernel<T, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); granted = smem; } \
        kernel<T, NT><<<dim3(n_experts, by_expert_row_blocks(rows, rows_per_warp, P, n_experts)), 256, smem, (cudaStream_t)stream>>>(__VA_ARGS__);         \
    })

extern "C" int ktb200_experts_gate_up_by_expert(const void* x, const int64_t* ids, int top, int n_experts, const void* w_gate, const void* w_up, void* act, int n_tokens, int width,
                                                int ff, int staged, int act_kind, float limit, int dtype, void* stream) {
    if (!x || !ids || !w_up || !act || top <= 0 || n_experts <= 0 || width <= 0 || ff <= 0 || act_kind < kActSilu || act_kind > kActClampedGlu) { set_error("experts_gate_up_by_expert: bad argument"); return KTB200_EINVAL; }
    if (n_tokens <= 0) return KTB200_OK;
    const int P = n_tokens * top;
    if (by_expert_staged(staged, P, n_experts) == 4) {
        constexpr int NT = 4;
        BY_EXPERT_LAUNCH(experts_gate_up_by_expert_kernel, ff, 2, (size_t)width, (const T*)x, ids, top, P, (const T*)w_gate, (const T*)w_up, (T*)act, width, ff, act_kind, limit);
    } else {
        constexpr int NT = 2;
        BY_EXPERT_LAUNCH(experts_gate_up_by_expert_kernel, ff, 2, (size_t)width, (const T*)x, ids, top, P, (const T*)w_gate, (const T*)w_up, (T*)act, width, ff, act_kind, limit);
    }
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}

extern "C" int ktb200_experts_down_by_expert(const void* act, const int64_t* ids, const float* weights, int top, int n_experts, const void* w_down, float* pair_rows, float* out,
                                             int n_tokens, int width, int ff, int staged, int dtype, void* stream) {
    if (!act || !ids || !weights || !w_down || !pair_rows || !out || top <= 0 || n_experts <= 0 || width <= 0 || ff <= 0) {
        set_error("experts_down_by_expert: bad argument");
        return KTB200_EINVAL;
    }
    if (n_tokens <= 0) return KTB200_OK;
    const int P = n_tokens * top;
    if (by_expert_staged(staged, P, n_experts) == 4) {
        constexpr int NT = 4;
        BY_EXPERT_LAUNCH(experts_down_by_expert_kernel, width, 4, (size_t)ff, (const T*)act, ids, P, (const T*)w_down, pair_rows, width, ff);
    } else {
        constexpr int NT = 2;
        BY_EXPERT_LAUNCH(experts_down_by_expert_kernel, width, 4, (size_t)ff, (const T*)act, ids, P, (const T*)w_down, pair_rows, width, ff);
    }
    KTB_LAUNCH_CHECK();
    const long n = (long)n_tokens * width;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    experts_combine_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(pair_rows, weights, top, out, n, width);
    KTB_LAUNCH_CHECK();
    return KTB200_OK;
}
