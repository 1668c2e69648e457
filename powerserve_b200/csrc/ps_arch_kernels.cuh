// ps_arch_kernels.cuh - device code of the layer-list model executor (ps_arch.cu).
//
// Tiled kernels (any batch width): one 64 x 64 x 16 fp32 tile core shared by the dense projections, the routed experts
// (rows gathered per expert), the attention scores (B operand = K cache rows) and P.V (B operand = V^T cache rows).
// Sequential blocks add one-CTA-per-token kernels around them: the seam between two sublayers (group or layer norm of the output,
// residual add, what a new pass of a looped model adds, norm of the sum), unit-RMS q / k with the value blend on the way into the cache,
// the latent attention's norms and rotations (half-split or neighbouring pairs).  Pooled windows: pa_k_pool_blocks forms the mean key /
// value of every block of positions that a batch completes; the scores / soft-max / P.V kernels take the blocks as further keys behind
// the tokens.  pa_k_dense_up1 is the first half of a feed-forward without a gate.
// The single-token kernels (bs == 1) live in ps_arch_decode.cuh.
#pragma once

#define PA_TM 64
#define PA_TN 64
#define PA_TK 16
#define PA_LD (PA_TM + 4)
#define PA_MAX_HEADS 64
#define PA_MAX_EXPERTS 256

// activation of a gated unit: PS_ACT_SWISH  g' sigmoid(alpha g') (u' + shift) on g' = min(g, limit), u' = clamp(u, +-limit)
//                             PS_ACT_GELU_TANH  the tanh form of gelu on g, times u
//                             PS_ACT_XIELU      one argument only: alpha z^2 + z / 2 above zero, shift (exp(z) - 1 - z) + z / 2 below
//                                               (alpha = softplus(p), shift = 1/2 + softplus(q) of the layer's two numbers)
struct PaAct {
    float limit, alpha, shift;
    int kind;
};

struct PaAttn {
    int H, G, dq, dv;
    float scale;
    const float *temp;      // [H] or null
    const float *rel;       // [rows][H] or null
    const uint16_t *bucket; // distance -> row, n_bucket entries
    int n_bucket;
    const float *mix;       // [H][H] or null
    int sink;               // the denominator has one more term ...
    const float *sink_v;    // ... exp(sink_v[h]) (null: exp(0))
    const float *r1, *r2;   // [H] each or null: score -= r1[h] * ln(1 + r2[h] * distance)
    int window;             // > 0: a query sees the keys at distances 0 .. window - 1 only
    int chunk;              // > 0: a query sees the keys of its own chunk of positions only (chunks counted from position 0)
    const float *lin;       // [H] or null: score -= lin[h] * distance
    // pool > 0 (with a window): one mean key / value per block of `pool` positions that lies wholly before the window.  The means sit
    // behind the token rows of the cache buffers (K: row n_ctx + b; V^T: [G * dv][n_pool] behind the token part); a query's pooled
    // scores sit at pool_off + b of its score row, the single-token step's block statistics from stat_off on
    int pool, n_pool, pool_off, stat_off;
    int n_ctx;
    int64_t ldS;            // row stride of the score rows
    int B;                  // rows per head in the score buffer (max_batch)
    float *pm, *pl;         // single-token step: per head and block of keys, max and sum of exponentials of the mixed scores
    int ldP;                // blocks per head in pm / pl
};

template <bool ROUND> __device__ __forceinline__ float pa_rnd(float v) {
    if (ROUND) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}
__device__ __forceinline__ float pa_ld(const bf16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ float pa_ld(const float *p) { return *p; }

// two weight rows against one fp32 vector, reduced over the warp (defined with the single-token kernels, ps_arch_decode.cuh)
template <bool ROUND>
__device__ __forceinline__ void pa_dot2(const bf16 *__restrict__ w0, const bf16 *__restrict__ w1, const float *x, int K, float xscale, int lane, float &s0, float &s1,
                                        int k_begin = 0, int k_end = -1);

// ---------------------------------------------------------------------------------------------------------------- tile core
// acc[i][j] += sum_k A(ty * 4 + i, k) * B(tx * 4 + j, k) for the CTA's 64 x 64 tile.  Every thread stages 4 k-values of ONE A
// row and ONE B row per step: `arow` / `brow` point at row (tid >> 2) of the tile (null = outside: zeros).
template <bool ROUND, typename BT, int NB>
__device__ __forceinline__ void pa_tile_mm(float (&acc)[NB][4][4], const float *arow, float ascale, const BT *brow0, const BT *brow1, int K, float (*As)[PA_LD],
                                           float (*Bs)[PA_TK][PA_LD]) {
    const int tid = threadIdx.x, lr = tid >> 2, kq = (tid & 3) * 4, tx = tid & 15, ty = tid >> 4;
    for (int k0 = 0; k0 < K; k0 += PA_TK) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int kk = k0 + kq + c;
            const bool in = kk < K;
            As[kq + c][lr] = (arow && in) ? pa_rnd<ROUND>(arow[kk] * ascale) : 0.f;
            Bs[0][kq + c][lr] = (brow0 && in) ? pa_ld(brow0 + kk) : 0.f;
            if (NB == 2) Bs[NB - 1][kq + c][lr] = (brow1 && in) ? pa_ld(brow1 + kk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < PA_TK; k++) {
            const float4 a4 = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[nb][k][tx * 4]);
                const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[nb][i][j] = fmaf(av[i], bv[j], acc[nb][i][j]);
            }
        }
        __syncthreads();
    }
}

#define PA_TILE_SMEM(NB)                          \
    __shared__ __align__(16) float As[PA_TK][PA_LD]; \
    __shared__ __align__(16) float Bs[NB][PA_TK][PA_LD]

// ---------------------------------------------------------------------------------------------------------------- small ops
// keep (null or [tokens][dim]) receives the same rows once more: the embedding output that later passes of a looped model add back
__global__ void __launch_bounds__(128) pa_k_embed(float *__restrict__ x, const bf16 *__restrict__ table, const int32_t *__restrict__ tokens, int dim, float scale,
                                                  float *__restrict__ keep) {
    const int t = blockIdx.x;
    const bf16 *row = table + (int64_t)tokens[t] * dim;
    float *out = x + (int64_t)t * dim;
    float *out2 = keep ? keep + (int64_t)t * dim : nullptr;
    if ((dim & 7) == 0) { // 16-byte loads: the whole row is in flight at once
        for (int c = threadIdx.x * 8; c < dim; c += blockDim.x * 8) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(row + c));
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float lo = __uint_as_float(u[i] << 16) * scale, hi = __uint_as_float(u[i] & 0xffff0000u) * scale;
                out[c + 2 * i] = lo;
                out[c + 2 * i + 1] = hi;
                if (out2) { out2[c + 2 * i] = lo; out2[c + 2 * i + 1] = hi; }
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        const float v = __bfloat162float(row[c]) * scale;
        out[c] = v;
        if (out2) out2[c] = v;
    }
}

// h = x / sqrt(mean(x^2) + eps) * w   (w already holds 1 + weight for unit-offset norms)
__global__ void __launch_bounds__(256) pa_k_norm(float *__restrict__ h, const float *__restrict__ x, const float *__restrict__ w, int dim, float eps) {
    __shared__ float red[8];
    __shared__ float inv_s;
    const float *xr = x + (int64_t)blockIdx.x * dim;
    float s = 0.f;
    for (int c = threadIdx.x; c < dim; c += 256) s = fmaf(xr[c], xr[c], s);
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; i++) t += red[i];
        inv_s = 1.0f / sqrtf(t / (float)dim + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    for (int c = threadIdx.x; c < dim; c += 256) h[(int64_t)blockIdx.x * dim + c] = xr[c] * inv * w[c];
}

// the batch's K rows go to kc[pos][:], its V rows transposed to vct[:][pos]
// (v_off: where the value rows start in a projected row - behind the keys, or AT the keys when the values are the keys)
__global__ void __launch_bounds__(256) pa_k_kv_store(const float *__restrict__ qkv, int ld, int qd, int kd, int vd, float *__restrict__ kc, float *__restrict__ vct, int n_ctx,
                                                     const int32_t *__restrict__ pos, int v_off) {
    const int t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    const int p = pos[t];
    const float *row = qkv + (int64_t)t * ld;
    if (c < kd) kc[(int64_t)p * kd + c] = row[qd + c];
    else if (c < kd + vd) vct[(int64_t)(c - kd) * n_ctx + p] = row[v_off + c - kd];
}

// The means of block b of `pool` positions: K row n_ctx + b and column b of the pooled V^T rows, each the sum of the block's cached
// entries in position order, divided by pool - so a mean does not depend on how the prompt was cut.  Channel c of kd + vd.
__device__ __forceinline__ void pa_pool_block(float *__restrict__ kc, float *__restrict__ vct, int kd, int vd, int n_ctx, int pool, int n_pool, int b, int c) {
    const int j0 = b * pool;
    float s = 0.f;
    if (c < kd) {
        for (int j = 0; j < pool; j++) s += kc[(int64_t)(j0 + j) * kd + c];
        kc[(int64_t)(n_ctx + b) * kd + c] = s / (float)pool;
    } else if (c < kd + vd) {
        const float *vr = vct + (int64_t)(c - kd) * n_ctx + j0;
        for (int j = 0; j < pool; j++) s += vr[j];
        vct[(int64_t)vd * n_ctx + (int64_t)(c - kd) * n_pool + b] = s / (float)pool;
    }
}
// the blocks that a batch completes (block b ends at position b pool + pool - 1).  Grid (channels / 256, candidate blocks); the
// batch's first position comes from device memory.
__global__ void __launch_bounds__(256) pa_k_pool_blocks(float *__restrict__ kc, float *__restrict__ vct, int kd, int vd, int n_ctx, int pool, int n_pool,
                                                        const int32_t *__restrict__ pos, int bs) {
    const int p0 = pos[0], b = p0 / pool + blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if ((int64_t)(b + 1) * pool > p0 + bs || (int64_t)(b + 1) * pool > n_ctx) return;
    pa_pool_block(kc, vct, kd, vd, n_ctx, pool, n_pool, b, c);
}

// x += mixer + sum of the feed-forward slots (fixed order)
__global__ void __launch_bounds__(256) pa_k_combine(float *__restrict__ x, const float *__restrict__ ao, const float *__restrict__ slot, int top, int dim) {
    const int t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= dim) return;
    float y = ao[(int64_t)t * dim + c];
    for (int r = 0; r < top; r++) y += slot[((int64_t)t * top + r) * dim + c];
    x[(int64_t)t * dim + c] += y;
}

// ---------------------------------------------------------------------------------------------------------------- sequential blocks
// block-wide sum over 256 threads, broadcast to all (two barriers)
__device__ __forceinline__ float pa_block_sum(float s, float *red) {
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads(); // red may still be read from the call before
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += red[i];
    return t;
}

// block-wide statistics of v[0 .. n) (each thread its own strided entries): mu = mean when `center`, else 0;
// returns 1 / sqrt(mean((v - mu)^2) + eps)
__device__ __forceinline__ float pa_block_stats(const float *v, int n, int center, float eps, float *red, float &mu) {
    mu = 0.f;
    if (center) {
        float m = 0.f;
        for (int c = threadIdx.x; c < n; c += 256) m += v[c];
        mu = pa_block_sum(m, red) / (float)n;
    }
    float s = 0.f;
    for (int c = threadIdx.x; c < n; c += 256) { const float d = v[c] - mu; s = fmaf(d, d, s); }
    return 1.0f / sqrtf(pa_block_sum(s, red) / (float)n + eps);
}

// The seam between two sublayers of a sequential block, one CTA per token:
//   y given:  x <- x + G(y; w_out)   (w_out null: x <- x + y)      the sublayer's output, normed, joins the residual stream
//   add_tok / add_vec given:  x <- x + add_tok[token] + add_vec     what a new pass of a looped model adds before its first layer
//   h given:  h  = G(x; w_in)                                       the next sublayer's input
// G cuts the vector into `groups` equal parts and divides each by its own sqrt(mean(part^2) + eps) before the weight; with
// `center` the part's mean is taken off first (a layer norm without bias).
__global__ void __launch_bounds__(256) pa_k_seam_norm(float *__restrict__ x, const float *__restrict__ y, const float *__restrict__ w_out, float *__restrict__ h,
                                                      const float *__restrict__ w_in, int dim, int groups, float eps, int center, const float *__restrict__ add_tok,
                                                      const float *__restrict__ add_vec) {
    __shared__ float red[8];
    const int64_t base = (int64_t)blockIdx.x * dim;
    const int gs = dim / groups;
    for (int g = 0; g < groups; g++) {
        const int c0 = g * gs;
        if (y) {
            float inv = 1.0f, mu = 0.f;
            if (w_out) inv = pa_block_stats(y + base + c0, gs, center, eps, red, mu);
            for (int c = threadIdx.x; c < gs; c += 256) x[base + c0 + c] += w_out ? (y[base + c0 + c] - mu) * inv * w_out[c0 + c] : y[base + c0 + c];
        }
        if (add_tok || add_vec)
            for (int c = threadIdx.x; c < gs; c += 256) x[base + c0 + c] += (add_tok ? add_tok[base + c0 + c] : 0.f) + (add_vec ? add_vec[c0 + c] : 0.f);
        if (h) {
            float mu;
            const float inv = pa_block_stats(x + base + c0, gs, center, eps, red, mu); // (a thread reads back its own writes)
            for (int c = threadIdx.x; c < gs; c += 256) h[base + c0 + c] = (x[base + c0 + c] - mu) * inv * w_in[c0 + c];
        }
    }
}

// warp-wide: 1 / sqrt(mean(v[0 .. n)^2) + eps)
__device__ __forceinline__ float pa_warp_inv_rms(const float *v, int n, float eps, int lane) {
    float s = 0.f;
    for (int c = lane; c < n; c += 32) s = fmaf(v[c], v[c], s);
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return 1.0f / sqrtf(s / (float)n + eps);
}

// After the q|k|v projection of a batch, one CTA per token: unit-RMS q heads (in place) and k heads (qk_norm), the value rows
// blended with the source layer's (v_mix), K row -> kc[pos][:], V row transposed -> vct[:][pos].
__global__ void __launch_bounds__(256) pa_k_qkv_post(float *__restrict__ qkv, int ld, int H, int G, int dq, int dv, int qk_norm, float eps, int v_mix,
                                                     const float *__restrict__ lambda, float *__restrict__ v_src, int ld_src, float *__restrict__ kc,
                                                     float *__restrict__ vct, int n_ctx, const int32_t *__restrict__ pos) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, p = pos[t];
    float *row = qkv + (int64_t)t * ld;
    const int qd = H * dq, kd = G * dq, vd = G * dv;
    for (int hh = warp; hh < H + G; hh += 8) { // q heads, then k heads
        float *v = row + hh * dq;
        const float inv = qk_norm ? pa_warp_inv_rms(v, dq, eps, lane) : 1.0f;
        if (hh < H) {
            if (qk_norm) for (int c = lane; c < dq; c += 32) v[c] *= inv;
        } else {
            float *dst = kc + (int64_t)p * kd + (hh - H) * dq;
            for (int c = lane; c < dq; c += 32) dst[c] = v[c] * inv;
        }
    }
    const float lam = v_mix == PS_VMIX_BLEND ? lambda[0] : 0.f;
    for (int c = threadIdx.x; c < vd; c += 256) {
        float v = row[qd + kd + c];
        if (v_mix == PS_VMIX_SOURCE) v_src[(int64_t)t * ld_src + c] = v;
        else if (v_mix == PS_VMIX_BLEND) v = (1.0f - lam) * v + lam * v_src[(int64_t)t * ld_src + c];
        vct[(int64_t)c * n_ctx + p] = v;
    }
}

// rotation of the first `dims` entries of a vector (pairs (i, i + dims / 2)) by the angles pos * freq[i], cos / sin times mscale.
// The product and its reduction to [-pi, pi] are formed in double (three operations), so that the float32 argument of cosf / sinf is
// good to 2e-7 at any position; a float32 product alone is off by pos * 6e-8.
struct PaRope {
    const double *freq; // [dims / 2]
    int dims;
    float mscale;
    int interleaved;    // pairs (2i, 2i + 1) instead of (i, i + dims / 2)
};
__device__ __forceinline__ void pa_rope_store(const PaRope &r, const float *src, float *dst, int n, int pos, int c) {
    const int half = r.dims >> 1;
    if (c >= r.dims) { if (c < n) dst[c] = src[c]; return; }
    const int i = r.interleaved ? c >> 1 : c < half ? c : c - half;
    const double turns = (double)pos * r.freq[i];
    const float ang = (float)fma(-rint(turns * 0.15915494309189535), 6.283185307179586, turns);
    const float cs = cosf(ang) * r.mscale, sn = sinf(ang) * r.mscale;
    if (r.interleaved) dst[c] = (c & 1) == 0 ? src[c] * cs - src[c + 1] * sn : src[c] * cs + src[c - 1] * sn;
    else dst[c] = c < half ? src[c] * cs - src[c + half] * sn : src[c] * cs + src[c - half] * sn;
}

// After the down-projections W_dq | W_dkv of a latent attention, one CTA per token.  Row t = [q latent (rq) | kv latent (rk) |
// rotated key part (dr)]: cq = N(q latent; wq) -> cq[t];  c = N(kv latent; wk) -> kc[pos][0 .. rk) and vct[.][pos];
// rot(key part, pos) -> kc[pos][rk .. rk + dr).
__global__ void __launch_bounds__(256) pa_k_latent_post(const float *__restrict__ t_in, int ld, int rq, int rk, int dr, const float *__restrict__ wq, const float *__restrict__ wk,
                                                        float eps, PaRope rope, float *__restrict__ cq, float *__restrict__ kc, float *__restrict__ vct, int n_ctx,
                                                        const int32_t *__restrict__ pos) {
    __shared__ float red[8];
    const int t = blockIdx.x, p = pos[t];
    const float *row = t_in + (int64_t)t * ld;
    float s = 0.f;
    for (int c = threadIdx.x; c < rq; c += 256) s = fmaf(row[c], row[c], s);
    const float iq = 1.0f / sqrtf(pa_block_sum(s, red) / (float)rq + eps);
    for (int c = threadIdx.x; c < rq; c += 256) cq[(int64_t)t * rq + c] = row[c] * iq * wq[c];
    s = 0.f;
    for (int c = threadIdx.x; c < rk; c += 256) s = fmaf(row[rq + c], row[rq + c], s);
    const float ik = 1.0f / sqrtf(pa_block_sum(s, red) / (float)rk + eps);
    float *krow = kc + (int64_t)p * (rk + dr);
    for (int c = threadIdx.x; c < rk; c += 256) {
        const float v = row[rq + c] * ik * wk[c];
        krow[c] = v;
        vct[(int64_t)c * n_ctx + p] = v;
    }
    for (int c = threadIdx.x; c < dr; c += 256) pa_rope_store(rope, row + rq + rk, krow + rk, dr, p, c);
}

// the rotated part of every query head: q[t][h * (dn + dr) + dn ..] -> qa[t][h * (rk + dr) + rk ..], rotated by the token's position
__global__ void __launch_bounds__(256) pa_k_rope_q(const float *__restrict__ q, float *__restrict__ qa, int H, int dn, int dr, int rk, PaRope rope, const int32_t *__restrict__ pos) {
    const int t = blockIdx.x, p = pos[t];
    for (int e = threadIdx.x; e < H * dr; e += 256) {
        const int hh = e / dr, c = e % dr;
        pa_rope_store(rope, q + ((int64_t)t * H + hh) * (dn + dr) + dn, qa + ((int64_t)t * H + hh) * (rk + dr) + rk, dr, p, c);
    }
}

// ---------------------------------------------------------------------------------------------------------------- dense
// C[m][n] = sum_k A[m][k] W[n][k] + bias[n].  blockIdx.z walks groups (per-head products): group z reads the columns of A from
// z * a_gs on, the matrix z of N x K weights, and writes the columns of C from z * c_gs on.
template <bool ROUND>
__global__ void __launch_bounds__(256) pa_k_linear(const float *__restrict__ A, int lda, const bf16 *__restrict__ W, const float *__restrict__ bias, float *__restrict__ C, int ldc,
                                                   int M, int N, int K, int a_gs = 0, int c_gs = 0) {
    PA_TILE_SMEM(1);
    const int tid = threadIdx.x, lr = tid >> 2, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * PA_TM, n0 = blockIdx.x * PA_TN;
    A += (int64_t)blockIdx.z * a_gs;
    C += (int64_t)blockIdx.z * c_gs;
    W += (int64_t)blockIdx.z * N * K;
    float acc[1][4][4] = {};
    const float *arow = (m0 + lr < M) ? A + (int64_t)(m0 + lr) * lda : nullptr;
    const bf16 *brow = (n0 + lr < N) ? W + (int64_t)(n0 + lr) * K : nullptr;
    pa_tile_mm<ROUND, bf16, 1>(acc, arow, 1.0f, brow, nullptr, K, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(int64_t)m * ldc + n] = acc[0][i][j] + (bias ? bias[n] : 0.f);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------- router
// how a router turns its logits into chosen experts and weights
struct PaRoute {
    int E, top;
    int act;           // PS_ROUTER_SIGMOID: every logit through a sigmoid; PS_ROUTER_SOFTMAX: soft-max over all experts
    int groups, keep;  // groups > 1: equal groups of neighbouring experts, a group is worth its best score, the `keep` best groups stay
    int renorm;        // the chosen scores are divided by their sum + eps
    float eps;
    int shared_gate;   // the router matrix has one more row: the logit of the shared expert's gate
};
// one thread: scores from the logits z, group limit, the top largest (ties: the lower expert) -> se / sw; sc is scratch of E entries,
// sw doubles as scratch of `groups` entries before it receives the weights
__device__ __forceinline__ void pa_route_serial(const float *__restrict__ z, const PaRoute &r, float *sc, int *se, float *sw) {
    const int E = r.E;
    if (r.act == PS_ROUTER_SOFTMAX) {
        float m = -INFINITY, sum = 0.f;
        for (int e = 0; e < E; e++) m = fmaxf(m, z[e]);
        for (int e = 0; e < E; e++) { sc[e] = expf(z[e] - m); sum += sc[e]; }
        const float inv = 1.0f / sum;
        for (int e = 0; e < E; e++) sc[e] *= inv;
    } else {
        for (int e = 0; e < E; e++) sc[e] = 1.0f / (1.0f + expf(-z[e]));
    }
    if (r.groups > 1) {
        const int per = E / r.groups;
        for (int g = 0; g < r.groups; g++) {
            float w = -1.f;
            for (int e = g * per; e < (g + 1) * per; e++) w = fmaxf(w, sc[e]);
            sw[g] = w;
        }
        for (int n = 0; n < r.keep; n++) { // the kept groups are marked by a worth of 2 (scores never exceed 1)
            int best = 0;
            float bv = -1.f;
            for (int g = 0; g < r.groups; g++)
                if (sw[g] <= 1.5f && sw[g] > bv) { bv = sw[g]; best = g; }
            sw[best] = 2.f;
        }
        for (int g = 0; g < r.groups; g++)
            if (sw[g] <= 1.5f)
                for (int e = g * per; e < (g + 1) * per; e++) sc[e] = -1.f;
    }
    float sum = 0.f;
    for (int n = 0; n < r.top; n++) {
        int best = 0;
        float bv = -1.f;
        for (int e = 0; e < E; e++)
            if (sc[e] > bv) { bv = sc[e]; best = e; }
        se[n] = best;
        sw[n] = bv;
        sum += bv;
        sc[best] = -2.f;
    }
    if (r.renorm)
        for (int n = 0; n < r.top; n++) sw[n] /= sum + r.eps;
}

// router logits W_r h in fp32 (h unrounded), then pa_route_serial -> sel_e / sel_w [token][top]; with a shared gate the matrix's
// last row gives sgate[token] = sigmoid(w_sg . h)
__global__ void __launch_bounds__(256) pa_k_router(const float *__restrict__ h, const bf16 *__restrict__ Wr, int dim, PaRoute r, int *__restrict__ sel_e,
                                                   float *__restrict__ sel_w, float *__restrict__ sgate) {
    __shared__ float zs[PA_MAX_EXPERTS + 1], sc[PA_MAX_EXPERTS], sw[PA_MAX_EXPERTS];
    __shared__ int se[PA_MAX_EXPERTS];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *hr = h + (int64_t)t * dim;
    const int n_rows = r.E + (r.shared_gate ? 1 : 0);
    for (int e = 2 * warp; e < n_rows; e += 16) { // a warp takes two rows at a time (16-byte loads where the width allows)
        const int e1 = min(e + 1, n_rows - 1);
        float s0, s1;
        pa_dot2<false>(Wr + (int64_t)e * dim, Wr + (int64_t)e1 * dim, hr, dim, 1.0f, lane, s0, s1);
        if (lane == 0) { zs[e] = s0; zs[e1] = s1; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        pa_route_serial(zs, r, sc, se, sw);
        for (int n = 0; n < r.top; n++) { sel_e[t * r.top + n] = se[n]; sel_w[t * r.top + n] = sw[n]; }
        if (r.shared_gate) sgate[t] = 1.0f / (1.0f + expf(-zs[r.E]));
    }
}

// (token, slot) pairs grouped by expert: row lists + the table of row tiles (tile_rows each, the last of an expert ragged) the expert kernels walk
__global__ void __launch_bounds__(256) pa_k_dispatch(const int *__restrict__ sel_e, const float *__restrict__ sel_w, int n, int top, int E, int tile_rows, int *__restrict__ row_token,
                                                     int *__restrict__ row_slot, float *__restrict__ row_w, int *__restrict__ tile_e, int *__restrict__ tile_row0,
                                                     int *__restrict__ tile_end, int *__restrict__ n_tiles) {
    __shared__ int cnt[PA_MAX_EXPERTS], off[PA_MAX_EXPERTS], fill[PA_MAX_EXPERTS];
    for (int e = threadIdx.x; e < E; e += 256) { cnt[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += 256) atomicAdd(&cnt[sel_e[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, nt = 0;
        for (int e = 0; e < E; e++) {
            off[e] = o;
            for (int r = 0; r < cnt[e]; r += tile_rows) { tile_e[nt] = e; tile_row0[nt] = o + r; tile_end[nt] = o + cnt[e]; nt++; }
            o += cnt[e];
        }
        *n_tiles = nt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += 256) {
        const int e = sel_e[i];
        const int p = off[e] + atomicAdd(&fill[e], 1);
        row_token[p] = i / top;
        row_slot[p] = i % top;
        row_w[p] = sel_w[i];
    }
}

__device__ __forceinline__ float pa_expert_act(float g, float u, PaAct act) {
    if (act.kind == PS_ACT_GELU_TANH) // 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * u
        return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    g = fminf(g, act.limit);
    u = fminf(fmaxf(u, -act.limit), act.limit);
    return g * (1.0f / (1.0f + expf(-act.alpha * g))) * (u + act.shift);
}

// the one-argument forms (a feed-forward without a gate)
__device__ __forceinline__ float pa_act1(float z, PaAct act) {
    if (act.kind == PS_ACT_XIELU) return z > 0.f ? fmaf(act.alpha * z, z, 0.5f * z) : fmaf(act.shift, expm1f(z) - z, 0.5f * z);
    if (act.kind == PS_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    z = fminf(z, act.limit);
    return z * (1.0f / (1.0f + expf(-act.alpha * z)));
}

// y[r][n] = act(gate_e . z_r, up_e . z_r), z_r = w_r * h[token_r] (route_on_input) or h[token_r]
template <bool ROUND>
__global__ void __launch_bounds__(256) pa_k_expert_up(const float *__restrict__ h, int ldh, const int *__restrict__ row_token, const float *__restrict__ row_w,
                                                      const int *__restrict__ tile_e, const int *__restrict__ tile_row0, const int *__restrict__ tile_end,
                                                      const int *__restrict__ n_tiles, const bf16 *__restrict__ Wg, const bf16 *__restrict__ Wu, float *__restrict__ y, int ff,
                                                      int dim, int on_input, PaAct act) {
    PA_TILE_SMEM(2);
    if ((int)blockIdx.y >= *n_tiles) return;
    const int tid = threadIdx.x, lr = tid >> 2, tx = tid & 15, ty = tid >> 4;
    const int e = tile_e[blockIdx.y], r0 = tile_row0[blockIdx.y], rend = tile_end[blockIdx.y], n0 = blockIdx.x * PA_TN;
    float acc[2][4][4] = {};
    const bool rin = r0 + lr < rend;
    const float *arow = rin ? h + (int64_t)row_token[r0 + lr] * ldh : nullptr;
    const float ascale = (rin && on_input) ? row_w[r0 + lr] : 1.0f;
    const int64_t wofs = ((int64_t)e * ff + n0 + lr) * dim;
    const bool nin = n0 + lr < ff;
    pa_tile_mm<ROUND, bf16, 2>(acc, arow, ascale, nin ? Wg + wofs : nullptr, nin ? Wu + wofs : nullptr, dim, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = r0 + ty * 4 + i;
        if (r >= rend) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < ff) y[(int64_t)r * ff + n] = pa_expert_act(acc[0][i][j], acc[1][i][j], act);
        }
    }
}

// slot[token_r][slot_r][n] = down_e . y_r  (times w_r when the score weighs the OUTPUT)
template <bool ROUND>
__global__ void __launch_bounds__(256) pa_k_expert_down(const float *__restrict__ y, int ff_ld, const int *__restrict__ row_token, const int *__restrict__ row_slot,
                                                        const float *__restrict__ row_w, const int *__restrict__ tile_e, const int *__restrict__ tile_row0,
                                                        const int *__restrict__ tile_end, const int *__restrict__ n_tiles, const bf16 *__restrict__ Wd, float *__restrict__ slot,
                                                        int top, int dim, int ff, int on_input) {
    PA_TILE_SMEM(1);
    if ((int)blockIdx.y >= *n_tiles) return;
    const int tid = threadIdx.x, lr = tid >> 2, tx = tid & 15, ty = tid >> 4;
    const int e = tile_e[blockIdx.y], r0 = tile_row0[blockIdx.y], rend = tile_end[blockIdx.y], n0 = blockIdx.x * PA_TN;
    float acc[1][4][4] = {};
    const float *arow = (r0 + lr < rend) ? y + (int64_t)(r0 + lr) * ff_ld : nullptr;
    const bf16 *brow = (n0 + lr < dim) ? Wd + ((int64_t)e * dim + n0 + lr) * ff : nullptr;
    pa_tile_mm<ROUND, bf16, 1>(acc, arow, 1.0f, brow, nullptr, ff, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = r0 + ty * 4 + i;
        if (r >= rend) continue;
        const float w = on_input ? 1.0f : row_w[r];
        float *dst = slot + ((int64_t)row_token[r] * top + row_slot[r]) * dim;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < dim) dst[n] = acc[0][i][j] * w;
        }
    }
}

// dense gated feed-forward, first half: y[m][n] = act(gate[n] . h_m, up[n] . h_m)
template <bool ROUND>
__global__ void __launch_bounds__(256) pa_k_dense_up(const float *__restrict__ h, int ldh, const bf16 *__restrict__ Wg, const bf16 *__restrict__ Wu, float *__restrict__ y, int M, int ff,
                                                     int dim, PaAct act) {
    PA_TILE_SMEM(2);
    const int tid = threadIdx.x, lr = tid >> 2, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * PA_TM, n0 = blockIdx.x * PA_TN;
    float acc[2][4][4] = {};
    const float *arow = (m0 + lr < M) ? h + (int64_t)(m0 + lr) * ldh : nullptr;
    const bool nin = n0 + lr < ff;
    pa_tile_mm<ROUND, bf16, 2>(acc, arow, 1.0f, nin ? Wg + (int64_t)(n0 + lr) * dim : nullptr, nin ? Wu + (int64_t)(n0 + lr) * dim : nullptr, dim, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < ff) y[(int64_t)m * ff + n] = pa_expert_act(acc[0][i][j], acc[1][i][j], act);
        }
    }
}

// feed-forward without a gate, first half: y[m][n] = act(up[n] . h_m)
template <bool ROUND>
__global__ void __launch_bounds__(256) pa_k_dense_up1(const float *__restrict__ h, int ldh, const bf16 *__restrict__ Wu, float *__restrict__ y, int M, int ff, int dim, PaAct act) {
    PA_TILE_SMEM(1);
    const int tid = threadIdx.x, lr = tid >> 2, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * PA_TM, n0 = blockIdx.x * PA_TN;
    float acc[1][4][4] = {};
    const float *arow = (m0 + lr < M) ? h + (int64_t)(m0 + lr) * ldh : nullptr;
    pa_tile_mm<ROUND, bf16, 1>(acc, arow, 1.0f, (n0 + lr < ff) ? Wu + (int64_t)(n0 + lr) * dim : nullptr, nullptr, dim, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < ff) y[(int64_t)m * ff + n] = pa_act1(acc[0][i][j], act);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------- attention
__device__ __forceinline__ float pa_score(const PaAttn &at, float dot, int h, int dist) {
    float s = dot * at.scale;
    if (at.temp) s *= at.temp[h];
    if (at.rel) s += at.rel[(int)at.bucket[min(dist, at.n_bucket - 1)] * at.H + h];
    if (at.r1) s -= at.r1[h] * logf(1.0f + at.r2[h] * (float)dist);
    if (at.lin) s -= at.lin[h] * (float)dist;
    return s;
}
// pooled blocks a query at position p sees: those that end at or before p - window
__device__ __forceinline__ int pa_pool_vis(const PaAttn &at, int p) { return (at.pool > 0 && p - at.window + 1 >= at.pool) ? (p - at.window + 1) / at.pool : 0; }
// first key a query at position p sees
__device__ __forceinline__ int pa_first_key(const PaAttn &at, int p) {
    int lo = at.window > 0 ? max(0, p - at.window + 1) : 0;
    if (at.chunk > 0) lo = max(lo, p - p % at.chunk);
    return lo;
}
__device__ __forceinline__ float pa_sink_logit(const PaAttn &at, int h) { return at.sink_v ? at.sink_v[h] : 0.f; }

// S[h][i][j] = score of query i (position pos[i]) and cache row j <= pos[i], before the heads are mixed.  Key tiles from
// `tok_tiles` on are tiles of pooled blocks: S[h][i][pool_off + b] = score of query i and the mean key of block b.
__global__ void __launch_bounds__(256) pa_k_scores(PaAttn at, const float *__restrict__ qkv, int ldq, const float *__restrict__ kc, int kd, float *__restrict__ S,
                                                   const int32_t *__restrict__ pos, int bs, int key_tile0, int tok_tiles) {
    PA_TILE_SMEM(1);
    const int tid = threadIdx.x, lr = tid >> 2, tx = tid & 15, ty = tid >> 4;
    const int h = blockIdx.z, g = h / (at.H / at.G), m0 = blockIdx.y * PA_TM;
    const int pos0 = pos[0], last = pos0 + min(m0 + PA_TM, bs) - 1; // the tile's furthest query
    if ((int)blockIdx.x >= tok_tiles) {
        const int b0 = ((int)blockIdx.x - tok_tiles) * PA_TN, nv = pa_pool_vis(at, last);
        if (b0 >= nv) return;
        float acc[1][4][4] = {};
        const float *arow = (m0 + lr < bs) ? qkv + (int64_t)(m0 + lr) * ldq + h * at.dq : nullptr;
        const float *brow = (b0 + lr < nv) ? kc + (int64_t)(at.n_ctx + b0 + lr) * kd + g * at.dq : nullptr;
        pa_tile_mm<false, float, 1>(acc, arow, 1.0f, brow, nullptr, at.dq, As, Bs);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int m = m0 + ty * 4 + i;
            if (m >= bs) continue;
            const int nvm = pa_pool_vis(at, pos0 + m);
            float *row = S + ((int64_t)h * at.B + m) * at.ldS + at.pool_off;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int b = b0 + tx * 4 + j;
                if (b < nvm) row[b] = acc[0][i][j] * at.scale * (at.temp ? at.temp[h] : 1.0f);
            }
        }
        return;
    }
    const int n0 = (blockIdx.x + key_tile0) * PA_TN;
    if (n0 > last || n0 + PA_TN <= pa_first_key(at, pos0 + m0)) return; // (the tile's first query sees furthest back)
    float acc[1][4][4] = {};
    const float *arow = (m0 + lr < bs) ? qkv + (int64_t)(m0 + lr) * ldq + h * at.dq : nullptr;
    const float *brow = (n0 + lr <= last) ? kc + (int64_t)(n0 + lr) * kd + g * at.dq : nullptr;
    pa_tile_mm<false, float, 1>(acc, arow, 1.0f, brow, nullptr, at.dq, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= bs) continue;
        const int p = pos0 + m;
        float *row = S + ((int64_t)h * at.B + m) * at.ldS;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n <= p && n >= pa_first_key(at, p)) row[n] = pa_score(at, acc[0][i][j], h, p - n);
        }
    }
}

// per query: mix the heads' scores (b_h = sum_g T[h][g] a_g), soft-max every head's row (optionally with a sink term in the
// denominator), zero the row's tail up to the end of the batch so that P.V can run whole tiles
template <int MAXH>
__device__ __forceinline__ void pa_mix_rows(const PaAttn &at, float *S, int i, int lo, int n, const float *Ts) {
    const int H = at.H;
    for (int j = lo + threadIdx.x; j < n; j += blockDim.x) {
        float a[MAXH];
#pragma unroll
        for (int g = 0; g < MAXH; g++) a[g] = g < H ? S[((int64_t)g * at.B + i) * at.ldS + j] : 0.f;
        for (int h = 0; h < H; h++) {
            float s = 0.f;
#pragma unroll
            for (int g = 0; g < MAXH; g++)
                if (g < H) s = fmaf(Ts[h * H + g], a[g], s);
            S[((int64_t)h * at.B + i) * at.ldS + j] = s;
        }
    }
}

__global__ void __launch_bounds__(256) pa_k_mix_softmax(PaAttn at, float *__restrict__ S, const int32_t *__restrict__ pos, int bs) {
    extern __shared__ float Ts[];
    const int i = blockIdx.x, H = at.H, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = pos[i] + 1, n_end = pos[0] + bs, lo = pa_first_key(at, pos[i]);
    const int lo_tile = pa_first_key(at, pos[0] + i / PA_TM * PA_TM); // P.V walks whole tiles of queries: from the tile's first key on
    if (at.mix) {
        for (int t = threadIdx.x; t < H * H; t += 256) Ts[t] = at.mix[t];
        __syncthreads();
        if (H <= 8) pa_mix_rows<8>(at, S, i, lo, n, Ts);
        else if (H <= 16) pa_mix_rows<16>(at, S, i, lo, n, Ts);
        else if (H <= 32) pa_mix_rows<32>(at, S, i, lo, n, Ts);
        else pa_mix_rows<PA_MAX_HEADS>(at, S, i, lo, n, Ts);
        __syncthreads();
    }
    // pooled blocks: the query's own, and those of its tile's furthest query (P.V walks whole tiles: zeros in between)
    const int nv = pa_pool_vis(at, pos[i]), nv_tile = pa_pool_vis(at, pos[0] + min(i / PA_TM * PA_TM + PA_TM, bs) - 1);
    for (int h = warp; h < H; h += 8) {
        float *row = S + ((int64_t)h * at.B + i) * at.ldS, *prow = row + at.pool_off;
        const float sk = pa_sink_logit(at, h);
        float mx = at.sink ? sk : -INFINITY;
        for (int j = lo + lane; j < n; j += 32) mx = fmaxf(mx, row[j]);
        for (int j = lane; j < nv; j += 32) mx = fmaxf(mx, prow[j]);
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
        for (int j = lo + lane; j < n; j += 32) {
            const float e = expf(row[j] - mx);
            row[j] = e;
            sum += e;
        }
        for (int j = lane; j < nv; j += 32) {
            const float e = expf(prow[j] - mx);
            prow[j] = e;
            sum += e;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (at.sink) sum += expf(sk - mx);
        const float inv = 1.0f / sum;
        for (int j = lo + lane; j < n; j += 32) row[j] *= inv;
        for (int j = n + lane; j < n_end; j += 32) row[j] = 0.f;
        for (int j = lo_tile + lane; j < lo; j += 32) row[j] = 0.f;
        for (int j = lane; j < nv; j += 32) prow[j] *= inv;
        for (int j = nv + lane; j < nv_tile; j += 32) prow[j] = 0.f;
    }
}

// att[i][h * dv + c] = sum_j P[h][i][j] V^T[g * dv + c][j]
__global__ void __launch_bounds__(256) pa_k_pv(PaAttn at, const float *__restrict__ S, const float *__restrict__ vct, float *__restrict__ att, int od,
                                               const int32_t *__restrict__ pos, int bs) {
    PA_TILE_SMEM(1);
    const int tid = threadIdx.x, lr = tid >> 2, tx = tid & 15, ty = tid >> 4;
    const int h = blockIdx.z, g = h / (at.H / at.G), m0 = blockIdx.y * PA_TM, n0 = blockIdx.x * PA_TN;
    const int n_keys = pos[0] + min(m0 + PA_TM, bs); // keys the tile's furthest query sees (the rows are zero beyond their own)
    const int k0 = pa_first_key(at, pos[0] + m0);    // ... and the first key its first query sees (zero before a row's own)
    float acc[1][4][4] = {};
    const float *arow = (m0 + lr < bs) ? S + ((int64_t)h * at.B + m0 + lr) * at.ldS + k0 : nullptr;
    const float *brow = (n0 + lr < at.dv) ? vct + (int64_t)(g * at.dv + n0 + lr) * at.n_ctx + k0 : nullptr;
    pa_tile_mm<false, float, 1>(acc, arow, 1.0f, brow, nullptr, n_keys - k0, As, Bs);
    const int nv = pa_pool_vis(at, n_keys - 1); // pooled blocks of the tile's furthest query: their weights times the mean value rows
    if (nv > 0) {
        const float *arow2 = (m0 + lr < bs) ? S + ((int64_t)h * at.B + m0 + lr) * at.ldS + at.pool_off : nullptr;
        const float *brow2 = (n0 + lr < at.dv) ? vct + (int64_t)at.G * at.dv * at.n_ctx + (int64_t)(g * at.dv + n0 + lr) * at.n_pool : nullptr;
        pa_tile_mm<false, float, 1>(acc, arow2, 1.0f, brow2, nullptr, nv, As, Bs);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= bs) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < at.dv) att[(int64_t)m * od + h * at.dv + n] = acc[0][i][j];
        }
    }
}
