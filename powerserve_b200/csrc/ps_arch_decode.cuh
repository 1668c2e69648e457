// ps_arch_decode.cuh - single-token (bs == 1) kernels of the layer-list executor: six launches per parallel block (seven per
// sequential block with windowed attention, eleven with latent attention), every one independent of the position except through
// device memory, so the step is captured once and replayed as a CUDA graph.
//
//   pa_k_dec_mv          weight-streaming mat-vec (bfloat16 rows, 16-byte loads, two rows per warp) with fused prologue / epilogue:
//                          norm of the residual stream in the prologue (q|k|v + router rows, lm_head),
//                          bias, K row / V^T column straight into the cache, router logits from the UNROUNDED fp32 input,
//                          residual add (output projection of a layer without a feed-forward);
//                          sequential blocks: the seam in the prologue (the pending sublayer output joins the residual stream through
//                          its group norm, the sum is group-normed for this product; CTA 0 stores the sum to the second residual buffer),
//                          per-head products (a row reads its head's slice of the input)
//   pa_k_dec_scores      scores of all heads for 16 keys per CTA (thread per key and head out of shared memory), distance bias (table,
//                        logarithmic or linear), head mixing, per-block soft-max statistics; with a window the grid starts at the first
//                        key in sight; pooled windows: further CTAs take 16 block means each, and the last CTA forms the mean of the
//                        block that the token completes
//   pa_k_dec_pv          soft-max statistics (+ sink logit) per head, weights staged once per CTA, P.V along contiguous V^T rows; many
//                        heads over one kv head are split over blockIdx.z
//   pa_k_dec_dense_up    seam in the prologue, gate | up rows of a dense feed-forward (or of a shared expert, then with the router's
//                        logits as further rows), activation; without a gate a warp's pair is two neighbouring up rows
//   pa_k_dec_expert_up   norm + top-k of the router scores in the prologue, gate | up rows of the chosen experts, activation
//   pa_k_dec_expert_down down rows of the chosen experts summed over the slots + mixer output + residual
#pragma once
#include "ps_ptx.cuh"

#define PA_DV_THREADS 256
#define PA_DV_ROWS 16       // output rows per mat-vec CTA: 8 warps x 2 rows
#define PA_DS_KEYS 16       // keys per CTA of the decode scores kernel
#define PA_DP_DIMS 4        // value dims per CTA of the decode P.V kernel (two warps each)
#define PA_DP_FLOATS 10240  // staged floats per CTA of the P.V kernel: (PA_DP_DIMS + heads per kv head) x chunk keys

// two rows at once: s0 += w0 . f(x), s1 += w1 . f(x) with f = bfloat16 rounding (ROUND) of x * xscale, or identity
template <bool ROUND>
__device__ __forceinline__ void pa_dot2(const bf16 *__restrict__ w0, const bf16 *__restrict__ w1, const float *x, int K, float xscale, int lane, float &s0, float &s1,
                                        int k_begin, int k_end) {
    s0 = s1 = 0.f;
    if (k_end < 0) k_end = K;
    if ((K & 7) == 0 && (k_begin & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) { // (a head's slice of x may start anywhere)
#pragma unroll 4
        for (int k = k_begin + lane * 8; k < k_end; k += 256) {
            const uint4 a = __ldg(reinterpret_cast<const uint4 *>(w0 + k));
            const uint4 b = __ldg(reinterpret_cast<const uint4 *>(w1 + k));
            const float4 x0 = *reinterpret_cast<const float4 *>(x + k), x1 = *reinterpret_cast<const float4 *>(x + k + 4);
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int t = 0; t < 4; t++) {
                const float xa = pa_rnd<ROUND>(xv[2 * t] * xscale), xb = pa_rnd<ROUND>(xv[2 * t + 1] * xscale);
                s0 = fmaf(__uint_as_float(au[t] << 16), xa, s0);
                s0 = fmaf(__uint_as_float(au[t] & 0xffff0000u), xb, s0);
                s1 = fmaf(__uint_as_float(bu[t] << 16), xa, s1);
                s1 = fmaf(__uint_as_float(bu[t] & 0xffff0000u), xb, s1);
            }
        }
    } else {
        for (int k = k_begin + lane; k < k_end; k += 32) {
            const float xa = pa_rnd<ROUND>(x[k] * xscale);
            s0 = fmaf(__bfloat162float(w0[k]), xa, s0);
            s1 = fmaf(__bfloat162float(w1[k]), xa, s1);
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) { s0 += __shfl_xor_sync(0xffffffffu, s0, o); s1 += __shfl_xor_sync(0xffffffffu, s1, o); }
}

// ask L2 for a warp's slice of two weight rows before the prologue's barriers: the stream then starts from L2
__device__ __forceinline__ void pa_prefetch2(const bf16 *w0, const bf16 *w1, int k_begin, int k_end, int lane) {
    for (int k = k_begin + lane * 64; k < k_end; k += 32 * 64) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(w0 + k));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(w1 + k));
    }
}

// block-wide: hs[k] = x[k] / sqrt(mean(x^2) + eps) * w[k]  (w holds 1 + weight for unit-offset norms); 256 threads
__device__ __forceinline__ void pa_norm_to_smem(float *hs, const float *__restrict__ x, const float *__restrict__ w, int dim, float eps) {
    __shared__ float red[8];
    __shared__ float inv_s;
    float s = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) s = fmaf(x[c], x[c], s);
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += red[i];
        inv_s = 1.0f / sqrtf(t / (float)dim + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) hs[c] = x[c] * inv * w[c];
    __syncthreads();
}

// block-wide seam of a sequential block (256 threads): hs = G(x + P(y) + add_tok + add_vec; w_in) with P(y) = G(y; w_out) (w_out
// null: y itself; y / add_tok / add_vec null: nothing joins), G over `groups` equal parts, the part's mean taken off first when
// `center`.  CTA 0 also stores the updated residual to x_out - a buffer other than x, which the other CTAs are still reading.
__device__ __forceinline__ void pa_seam_to_smem(float *hs, const float *__restrict__ x, const float *__restrict__ y, const float *__restrict__ w_out,
                                                const float *__restrict__ w_in, float *__restrict__ x_out, int dim, int groups, float eps, int center = 0,
                                                const float *__restrict__ add_tok = nullptr, const float *__restrict__ add_vec = nullptr) {
    __shared__ float red[8];
    const int gs = dim / groups;
    for (int g = 0; g < groups; g++) {
        const int c0 = g * gs;
        float inv = 1.0f, mu = 0.f;
        if (y && w_out) inv = pa_block_stats(y + c0, gs, center, eps, red, mu);
        for (int c = threadIdx.x; c < gs; c += 256) {
            float v = x[c0 + c];
            if (y) v += w_out ? (y[c0 + c] - mu) * inv * w_out[c0 + c] : y[c0 + c];
            if (add_tok || add_vec) v += (add_tok ? add_tok[c0 + c] : 0.f) + (add_vec ? add_vec[c0 + c] : 0.f);
            hs[c0 + c] = v;
            if (x_out && blockIdx.x == 0 && blockIdx.y == 0) x_out[c0 + c] = v;
        }
        if (w_in) {
            float mu2;
            const float inv2 = pa_block_stats(hs + c0, gs, center, eps, red, mu2); // (a thread's own entries)
            for (int c = threadIdx.x; c < gs; c += 256) hs[c0 + c] = (hs[c0 + c] - mu2) * inv2 * w_in[c0 + c];
        }
    }
    __syncthreads();
}

struct PaMv {
    const float *x;        // input vector [K]
    const float *norm_w;   // non-null: the input is normed first (K = model width)
    float eps;
    // sequential blocks (groups > 0): the input is the seam G(x + P(seam_y; seam_w); norm_w); CTA 0 stores x + P(..) to x_out
    int groups;
    const float *seam_y, *seam_w;
    float *x_out;
    int center;            // the norms take the mean off first
    const float *add_tok, *add_vec; // what a new pass of a looped model adds to the stream at this seam (null: nothing)
    // per-head products (grp_rows > 0): rows [g * grp_rows, (g + 1) * grp_rows) read x + g * x_gs and write y + g * y_gs
    int grp_rows, x_gs, y_gs;
    const bf16 *W;         // [N][K]
    const float *bias;     // [N] or null
    int N, K;
    float *y;              // [N] (rows routed to the cache below are not stored here)
    float *residual;       // non-null: residual[n] += result instead of y[n] = result
    // q | k | v routing of the rows: [0, qd) -> y, [qd, qd + kd) -> K cache row `pos`, then vd rows -> V^T column `pos` (kd = 0: none)
    int qd, kd, vd;
    float *kc, *vct;
    int n_ctx;
    const int32_t *pos;
    int v_is_k;            // the K rows are the value rows as well: each goes to the K cache row AND to its V^T column (vd = 0)
    // extra fp32-input rows after the N weight rows: router logits z[e] = Wr[e] . h (h unrounded)
    const bf16 *Wr;
    int E;
    float *z;
    int ksplit;            // warps of a CTA that share a row pair, each taking K / ksplit of the columns (1, 2, 4 or 8)
    int prefetch;          // 1: request the first row group into L2 before the dependency wait; 2: also every next group one ahead
};

template <bool ROUND>
__global__ void __launch_bounds__(PA_DV_THREADS) pa_k_dec_mv(const PaMv a) {
    extern __shared__ __align__(16) float pa_hs[];
    __shared__ float part_s[8][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ks = a.ksplit, pairs = 8 / ks, pair = warp % pairs, slice = warp / pairs;
    const int total = a.N + a.E;
    const int groups = (total + 2 * pairs - 1) / (2 * pairs); // row groups of `pairs` row pairs; the CTAs walk them with the grid's stride
    const int kc = a.K / ks, k_begin = slice * kc, k_end = slice == ks - 1 ? a.K : k_begin + kc;
    // rows of a pair: weight rows below N, router rows (fp32 input, never rounded) from N on
    auto row = [&](int n) { return n < a.N ? a.W + (int64_t)n * a.K : a.Wr + (int64_t)(n - a.N) * a.K; };
    auto prefetch = [&](int grp) {
        const int n0 = (grp * pairs + pair) * 2;
        if (a.prefetch && n0 < total) pa_prefetch2(row(n0), row(min(n0 + 1, total - 1)), k_begin, k_end, lane);
    };
    prefetch(blockIdx.x);
    // launched with programmatic stream serialisation: everything above touches weights only and overlaps the kernel before
    ps_grid_dep_launch();
    ps_grid_dep_wait();
    const float *xin = a.x;
    if (a.groups > 0) {
        pa_seam_to_smem(pa_hs, a.x, a.seam_y, a.seam_w, a.norm_w, a.x_out, a.K, a.groups, a.eps, a.center, a.add_tok, a.add_vec);
        xin = pa_hs;
    } else if (a.norm_w) {
        pa_norm_to_smem(pa_hs, a.x, a.norm_w, a.K, a.eps);
        xin = pa_hs;
    }
    for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
        if (a.prefetch > 1 && grp + (int)gridDim.x < groups) prefetch(grp + gridDim.x); // opt-in: the next group's rows travel to L2 meanwhile
        const int n0 = (grp * pairs + pair) * 2, n1 = min(n0 + 1, total - 1);
        const bool live = n0 < total;
        float s0 = 0.f, s1 = 0.f;
        if (live) {
            const bf16 *w0 = row(n0), *w1 = row(n1);
            if (a.grp_rows > 0) { // every row reads its own head's slice of x
                float t;
                pa_dot2<ROUND>(w0, w0, xin + (n0 / a.grp_rows) * a.x_gs, a.K, 1.0f, lane, s0, t, k_begin, k_end);
                pa_dot2<ROUND>(w1, w1, xin + (n1 / a.grp_rows) * a.x_gs, a.K, 1.0f, lane, s1, t, k_begin, k_end);
            } else if (n0 >= a.N) {
                pa_dot2<false>(w0, w1, xin, a.K, 1.0f, lane, s0, s1, k_begin, k_end);
            } else if (n1 >= a.N) { // the pair straddles the two matrices
                float t;
                pa_dot2<ROUND>(w0, w0, xin, a.K, 1.0f, lane, s0, t, k_begin, k_end);
                pa_dot2<false>(w1, w1, xin, a.K, 1.0f, lane, s1, t, k_begin, k_end);
            } else {
                pa_dot2<ROUND>(w0, w1, xin, a.K, 1.0f, lane, s0, s1, k_begin, k_end);
            }
        }
        if (ks > 1) {
            if (lane == 0) { part_s[warp][0] = s0; part_s[warp][1] = s1; }
            __syncthreads();
            if (slice == 0) {
                s0 = s1 = 0.f;
                for (int q = 0; q < ks; q++) { s0 += part_s[q * pairs + pair][0]; s1 += part_s[q * pairs + pair][1]; }
            }
        }
        if (slice == 0 && live && lane < 2 && !(lane && n1 == n0)) {
            const int n = lane ? n1 : n0;
            float v = lane ? s1 : s0;
            if (n >= a.N) {
                a.z[n - a.N] = v;
            } else {
                if (a.bias) v += a.bias[n];
                if (a.kd && n >= a.qd && n < a.qd + a.kd + a.vd) {
                    const int p = a.pos[0];
                    if (n < a.qd + a.kd) {
                        a.kc[(int64_t)p * a.kd + (n - a.qd)] = v;
                        if (a.v_is_k) a.vct[(int64_t)(n - a.qd) * a.n_ctx + p] = v;
                    } else {
                        a.vct[(int64_t)(n - a.qd - a.kd) * a.n_ctx + p] = v;
                    }
                } else if (a.residual) {
                    a.residual[n] += v;
                } else if (a.grp_rows > 0) {
                    a.y[(n / a.grp_rows) * a.y_gs + n % a.grp_rows] = v;
                } else {
                    a.y[n] = v;
                }
            }
        }
        if (ks > 1) __syncthreads(); // part_s is written again by the next group
    }
}

// ---------------------------------------------------------------------------------------------------- decode attention
// b[h][j] for the CTA's PA_DS_KEYS keys.  The keys' cache rows arrive in shared memory by 1-D bulk copies (one per row, the rows
// padded against bank conflicts) while the threads fetch q; then a thread per (key, head) forms the dot product with float4 reads
// and applies scale / temperature / distance bias - no shuffles, and the bias look-ups of all pairs are in flight together.
// CTAs from `tok_blocks` on take 16 pooled blocks each: the mean key rows behind the token rows, scores at pool_off, statistics at stat_off.
// With pool_v given, the last CTA also forms the means of the block that this token completes (no query sees that block before a
// later step, so nothing in this launch reads them).
__global__ void __launch_bounds__(256) pa_k_dec_scores(PaAttn at, const float *__restrict__ q, const float *kc, const int32_t *__restrict__ pos_dev,
                                                       float *__restrict__ b, int *__restrict__ err, int tok_blocks, float *pool_v) {
    extern __shared__ __align__(16) float sm[];
    __shared__ __align__(8) uint64_t bar;
    const int H = at.H, G = at.G, dq = at.dq, rep = H / G, kd = G * dq, kds = ((kd + 3) & ~3) + 4;
    float *ks = sm;                        // [PA_DS_KEYS][kds]
    float *qs = ks + PA_DS_KEYS * kds;     // [H][dq]
    float *sa = qs + H * dq;               // [H][PA_DS_KEYS + 1]
    float *Ts = sa + H * (PA_DS_KEYS + 1); // [H][H]
    const int tid = threadIdx.x;
    if (at.mix) for (int t = tid; t < H * H; t += 256) Ts[t] = at.mix[t]; // a weight: fetched before the dependency wait
    ps_grid_dep_launch();
    ps_grid_dep_wait();
    const int pos = pos_dev[0];
    if (pool_v && at.pool > 0 && blockIdx.x == gridDim.x - 1 && (pos + 1) % at.pool == 0 && pos + 1 <= at.n_ctx)
        for (int c = tid; c < kd + G * at.dv; c += 256) pa_pool_block(const_cast<float *>(kc), pool_v, kd, G * at.dv, at.n_ctx, at.pool, at.n_pool, (pos + 1) / at.pool - 1, c);
    const bool pooled = (int)blockIdx.x >= tok_blocks;
    int lo = pa_first_key(at, pos);
    int blk = lo / PA_DS_KEYS + blockIdx.x, j0 = blk * PA_DS_KEYS; // the grid starts at the block of the first key in sight
    int nj = min(PA_DS_KEYS, pos + 1 - j0), s_off = 0;
    if (pooled) { // rows n_ctx + j0 .. of the K buffer; every one of the first pa_pool_vis blocks is in sight
        lo = 0;
        j0 = ((int)blockIdx.x - tok_blocks) * PA_DS_KEYS;
        nj = min(PA_DS_KEYS, pa_pool_vis(at, pos) - j0);
        blk = at.stat_off + (int)blockIdx.x - tok_blocks;
        s_off = at.pool_off;
        kc += (int64_t)at.n_ctx * kd;
    }
    if (nj <= 0) return;
    const bool bulk = (kd & 3) == 0;
    if (bulk && tid == 0) {
        ps_mbar_init(&bar, 1);
        ps_fence_barrier_init();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        ps_mbar_expect_tx(&bar, (uint32_t)(nj * kd * 4));
        for (int jj = 0; jj < nj; jj++) ps_bulk_g2s(ks + jj * kds, kc + (int64_t)(j0 + jj) * kd, (uint32_t)(kd * 4), &bar);
    }
    if (!bulk) for (int t = tid; t < nj * kd; t += 256) ks[(t / kd) * kds + t % kd] = kc[(int64_t)j0 * kd + t];
    for (int t = tid; t < H * dq; t += 256) qs[t] = q[t];
    __syncthreads();
    if (bulk && !ps_tc_wait(&bar, 0)) { if (tid == 0) err[0] = 5; return; }
    for (int t = tid; t < PA_DS_KEYS * H; t += 256) {
        const int jj = t % PA_DS_KEYS, h = t / PA_DS_KEYS;
        if (jj >= nj || j0 + jj < lo) continue;
        const float *kr = ks + jj * kds + (h / rep) * dq, *qr = qs + h * dq;
        float s;
        if ((dq & 3) == 0) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int d = 0; d < dq; d += 4) {
                const float4 k4 = *reinterpret_cast<const float4 *>(kr + d), q4 = *reinterpret_cast<const float4 *>(qr + d);
                acc.x = fmaf(k4.x, q4.x, acc.x); acc.y = fmaf(k4.y, q4.y, acc.y); acc.z = fmaf(k4.z, q4.z, acc.z); acc.w = fmaf(k4.w, q4.w, acc.w);
            }
            s = (acc.x + acc.y) + (acc.z + acc.w);
        } else {
            s = 0.f;
            for (int d = 0; d < dq; d++) s = fmaf(kr[d], qr[d], s);
        }
        sa[h * (PA_DS_KEYS + 1) + jj] = pa_score(at, s, h, pooled ? 0 : pos - (j0 + jj));
    }
    __syncthreads();
    // mix the heads, store, and leave the block's soft-max statistics (max, sum of exponentials) for the P.V kernel:
    // the 16 keys of a head sit in 16 adjacent lanes
    const int n_t = (PA_DS_KEYS * H + 31) & ~31;
    for (int t = tid; t < n_t; t += 256) {
        const int h = t / PA_DS_KEYS, jj = t % PA_DS_KEYS;
        const bool valid = h < H && jj < nj && j0 + jj >= lo;
        float s = -INFINITY;
        if (valid) {
            if (at.mix) {
                s = 0.f;
                for (int g = 0; g < H; g++) s = fmaf(Ts[h * H + g], sa[g * (PA_DS_KEYS + 1) + jj], s);
            } else {
                s = sa[h * (PA_DS_KEYS + 1) + jj];
            }
            b[(int64_t)h * at.ldS + s_off + j0 + jj] = s;
        }
        float m = s;
#pragma unroll
        for (int o = PA_DS_KEYS / 2; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float e = valid ? expf(s - m) : 0.f;
#pragma unroll
        for (int o = PA_DS_KEYS / 2; o; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
        if (h < H && jj == 0) { // (every lane of the 16 holds the block's pair; the block has a key in sight)
            at.pm[(int64_t)h * at.ldP + blk] = m;
            at.pl[(int64_t)h * at.ldP + blk] = e;
        }
    }
}

// att[h][c] = sum_j p_hj V^T[g(h) dv + c][j] for one kv head g and PA_DP_DIMS value dims; p = soft-max of b[h][0 .. pos] with the
// optional sink term.  Phase 1: max and sum of every query head of the group, merged from the per-block pairs the scores kernel
// left (16 keys each).  Phase 2, per chunk of keys: the CTA's V^T rows
// arrive by 1-D bulk copies while the threads compute the chunk's weights once into shared memory; two warps per value dim
// (the halves of the chunk) then run float4 dot products out of shared memory for every head of the group.
__global__ void __launch_bounds__(256) pa_k_dec_pv(PaAttn at, const float *__restrict__ b, const float *__restrict__ vct, const int32_t *__restrict__ pos_dev,
                                                   float *__restrict__ att, int chunk, int *__restrict__ err) {
    extern __shared__ __align__(16) float sm[];
    __shared__ __align__(8) uint64_t bar;
    // blockIdx.z splits the query heads that share kv head g (many heads over one latent): this CTA takes `rep` of them from h0 on
    const int H = at.H, G = at.G, dv = at.dv, rep_all = H / G, g = blockIdx.y;
    const int rep_z = (rep_all + (int)gridDim.z - 1) / (int)gridDim.z, h0 = g * rep_all + (int)blockIdx.z * rep_z, rep = min(rep_z, rep_all - (int)blockIdx.z * rep_z);
    if (rep <= 0) return;
    float *vs = sm;                         // [PA_DP_DIMS][chunk] V^T rows of the chunk
    float *ps = vs + PA_DP_DIMS * chunk;    // [rep][chunk] soft-max weights of the chunk (un-normalised)
    float *ms = ps + rep * chunk;           // [rep] row maxima
    float *inv = ms + rep;                  // [rep] 1 / denominators
    float *acc = inv + rep;                 // [8 warps][rep]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    ps_grid_dep_launch();
    ps_grid_dep_wait();
    const int n = pos_dev[0] + 1, lo = pa_first_key(at, n - 1);
    const bool bulk = (at.n_ctx & 3) == 0;
    if (bulk && tid == 0) {
        ps_mbar_init(&bar, 1);
        ps_fence_barrier_init();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // soft-max statistics of every head of the group from the scores kernel's per-block pairs: a warp per head
    const int nb = (n + PA_DS_KEYS - 1) / PA_DS_KEYS;
    const int nv = pa_pool_vis(at, n - 1), nvb = (nv + PA_DS_KEYS - 1) / PA_DS_KEYS; // pooled blocks in sight, and their statistics
    for (int r = warp; r < rep; r += 8) {
        const float *bm = at.pm + (int64_t)(h0 + r) * at.ldP, *bl = at.pl + (int64_t)(h0 + r) * at.ldP;
        const float sk = pa_sink_logit(at, h0 + r);
        float mx = at.sink ? sk : -INFINITY;
        for (int j = lo / PA_DS_KEYS + lane; j < nb; j += 32) mx = fmaxf(mx, bm[j]);
        for (int j = lane; j < nvb; j += 32) mx = fmaxf(mx, bm[at.stat_off + j]);
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
        for (int j = lo / PA_DS_KEYS + lane; j < nb; j += 32) sum = fmaf(bl[j], expf(bm[j] - mx), sum);
        for (int j = lane; j < nvb; j += 32) sum = fmaf(bl[at.stat_off + j], expf(bm[at.stat_off + j] - mx), sum);
#pragma unroll
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) {
            if (at.sink) sum += expf(sk - mx);
            ms[r] = mx;
            inv[r] = 1.0f / sum;
        }
    }
    for (int t = tid; t < 8 * rep; t += 256) acc[t] = 0.f;
    const int dim_l = warp % PA_DP_DIMS, part = warp / PA_DP_DIMS, n_part = 8 / PA_DP_DIMS;
    const int c0 = blockIdx.x * PA_DP_DIMS;
    int it = 0;
    // two stretches of keys: the tokens in sight (V^T rows of n_ctx columns), then the pooled blocks (rows of n_pool columns behind them)
    for (int seg = 0; seg < (nv > 0 ? 2 : 1); seg++) {
    const float *vbase = seg ? vct + (int64_t)G * dv * at.n_ctx : vct;
    const int ldv = seg ? at.n_pool : at.n_ctx, s_lo = seg ? 0 : lo, s_n = seg ? nv : n, s_off = seg ? at.pool_off : 0;
    for (int j0 = s_lo & ~3; j0 < s_n; j0 += chunk, it++) { // (bulk copies start on 16-byte boundaries)
        const int nj = min(chunk, s_n - j0), nj4 = (nj + 3) & ~3;
        __syncthreads(); // the previous chunk's buffers are free
        if (bulk) {
            if (tid == 0) {
                const int rows = min(PA_DP_DIMS, dv - c0);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the rows were read through the generic proxy
                ps_mbar_expect_tx(&bar, (uint32_t)(rows * nj4 * 4));
                for (int cc = 0; cc < rows; cc++) ps_bulk_g2s(vs + cc * chunk, vbase + (int64_t)(g * dv + c0 + cc) * ldv + j0, (uint32_t)(nj4 * 4), &bar);
            }
        } else {
            for (int t = tid; t < PA_DP_DIMS * nj4; t += 256) {
                const int cc = t / nj4, jj = t % nj4;
                vs[cc * chunk + jj] = (c0 + cc < dv && jj < nj) ? vbase[(int64_t)(g * dv + c0 + cc) * ldv + j0 + jj] : 0.f;
            }
        }
        for (int t = tid; t < rep * nj4; t += 256) {
            const int r = t / nj4, jj = t % nj4;
            ps[r * chunk + jj] = (jj < nj && j0 + jj >= s_lo) ? expf(b[(int64_t)(h0 + r) * at.ldS + s_off + j0 + jj] - ms[r]) : 0.f;
        }
        __syncthreads();
        if (bulk && !ps_tc_wait(&bar, it & 1)) { if (tid == 0) err[0] = 6; return; }
        if (c0 + dim_l < dv) {
            const float4 *v4 = reinterpret_cast<const float4 *>(vs + dim_l * chunk);
            for (int r = 0; r < rep; r++) {
                const float4 *p4 = reinterpret_cast<const float4 *>(ps + r * chunk);
                float s = 0.f;
                for (int i = lane + 32 * part; i < nj4 / 4; i += 32 * n_part) {
                    const float4 v = v4[i], p = p4[i];
                    s = fmaf(p.x, v.x, s); s = fmaf(p.y, v.y, s); s = fmaf(p.z, v.z, s); s = fmaf(p.w, v.w, s);
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) acc[warp * rep + r] += s;
            }
        }
    }
    }
    __syncthreads();
    for (int t = tid; t < PA_DP_DIMS * rep; t += 256) {
        const int cc = t / rep, r = t % rep;
        if (c0 + cc >= dv) continue;
        float s = 0.f;
        for (int pp = 0; pp < n_part; pp++) s += acc[(pp * PA_DP_DIMS + cc) * rep + r];
        att[(h0 + r) * dv + c0 + cc] = s * inv[r];
    }
}

// ---------------------------------------------------------------------------------------------------- routed experts
// grid (row pairs of ff, top_k): y[r][n] = act(gate_e . z, up_e . z), z = round(w_r * h) (score on the input) or round(h)
template <bool ROUND>
__global__ void __launch_bounds__(PA_DV_THREADS) pa_k_dec_expert_up(const float *__restrict__ x, const float *__restrict__ norm_w, float eps, const float *__restrict__ z, PaRoute rt,
                                                                    const bf16 *__restrict__ Wg, const bf16 *__restrict__ Wu, float *__restrict__ y,
                                                                    int ff, int dim, int on_input, PaAct act, int *__restrict__ sel_e,
                                                                    float *__restrict__ sel_w) {
    extern __shared__ __align__(16) float pa_hs[];
    __shared__ float sc[PA_MAX_EXPERTS];
    __shared__ int se[PA_MAX_EXPERTS];
    __shared__ float sw[PA_MAX_EXPERTS];
    if (threadIdx.x == 0) {
        pa_route_serial(z, rt, sc, se, sw);
        if (blockIdx.x == 0 && blockIdx.y == 0)
            for (int r = 0; r < rt.top; r++) { sel_e[r] = se[r]; sel_w[r] = sw[r]; }
    }
    if (norm_w) {
        pa_norm_to_smem(pa_hs, x, norm_w, dim, eps); // (its barriers also publish se / sw)
    } else { // the experts read the residual stream itself
        for (int c = threadIdx.x; c < dim; c += blockDim.x) pa_hs[c] = x[c];
        __syncthreads();
    }
    const int r = blockIdx.y, e = se[r], lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float w = on_input ? sw[r] : 1.0f;
    // a warp owns one ff row at a time: its gate row and its up row are the pair; the CTAs walk the row groups with the grid's stride
    const int rows = PA_DV_ROWS / 2;
    for (int n = blockIdx.x * rows + warp; n < ff; n += gridDim.x * rows) {
        const bf16 *wg = Wg + ((int64_t)e * ff + n) * dim, *wu = Wu + ((int64_t)e * ff + n) * dim;
        float gsum, usum;
        pa_dot2<ROUND>(wg, wu, pa_hs, dim, w, lane, gsum, usum);
        if (lane == 0) y[(int64_t)r * ff + n] = pa_expert_act(gsum, usum, act);
    }
}

// dense gated feed-forward of a sequential block, first half: the seam in the prologue (the mixer's output joins the residual
// stream, the result is normed), then y[n] = act(gate[n] . h, up[n] . h); a warp owns one ff row at a time, the CTAs walk the row
// groups with the grid's stride
template <bool ROUND>
__global__ void __launch_bounds__(PA_DV_THREADS) pa_k_dec_dense_up(const float *__restrict__ x, const float *__restrict__ seam_y, const float *__restrict__ seam_w,
                                                                   const float *__restrict__ norm_w, float *__restrict__ x_out, int groups, float eps, const bf16 *__restrict__ Wg,
                                                                   const bf16 *__restrict__ Wu, float *__restrict__ y, int ff, int dim, PaAct act,
                                                                   const bf16 *__restrict__ Wr = nullptr, int E = 0, float *__restrict__ z = nullptr, int center = 0) {
    extern __shared__ __align__(16) float pa_hs[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, rows = PA_DV_ROWS / 2;
    if (!Wg) { // no gate: a warp's pair is two neighbouring up rows, y[n] = act(up[n] . h)
        const int n = (blockIdx.x * rows + warp) * 2;
        if (n < ff) pa_prefetch2(Wu + (int64_t)n * dim, Wu + (int64_t)min(n + 1, ff - 1) * dim, 0, dim, lane);
        ps_grid_dep_launch();
        ps_grid_dep_wait();
        pa_seam_to_smem(pa_hs, x, seam_y, seam_w, norm_w, x_out, dim, groups, eps, center);
        for (int n0 = (blockIdx.x * rows + warp) * 2; n0 < ff; n0 += gridDim.x * rows * 2) {
            const int n1 = min(n0 + 1, ff - 1);
            float s0, s1;
            pa_dot2<ROUND>(Wu + (int64_t)n0 * dim, Wu + (int64_t)n1 * dim, pa_hs, dim, 1.0f, lane, s0, s1);
            if (lane == 0) y[n0] = pa_act1(s0, act);
            if (lane == 1 && n1 != n0) y[n1] = pa_act1(s1, act);
        }
        return;
    }
    {
        const int n = blockIdx.x * rows + warp;
        if (n < ff) pa_prefetch2(Wg + (int64_t)n * dim, Wu + (int64_t)n * dim, 0, dim, lane);
    }
    ps_grid_dep_launch();
    ps_grid_dep_wait();
    pa_seam_to_smem(pa_hs, x, seam_y, seam_w, norm_w, x_out, dim, groups, eps, center);
    // E more rows behind the ff rows: a router's logits z[e] = Wr[e] . h from the UNROUNDED input (a shared expert's launch carries them)
    for (int n = blockIdx.x * rows + warp; n < ff + E; n += gridDim.x * rows) {
        float gsum, usum;
        if (n >= ff) {
            const bf16 *wr = Wr + (int64_t)(n - ff) * dim;
            pa_dot2<false>(wr, wr, pa_hs, dim, 1.0f, lane, gsum, usum);
            if (lane == 0) z[n - ff] = gsum;
            continue;
        }
        pa_dot2<ROUND>(Wg + (int64_t)n * dim, Wu + (int64_t)n * dim, pa_hs, dim, 1.0f, lane, gsum, usum);
        if (lane == 0) y[n] = pa_expert_act(gsum, usum, act);
    }
}

// x[n] += ao[n] + sum_r down_{e_r}[n] . round(y_r)  (times w_r when the score weighs the output); slots in order; `ksplit`
// warps share a row pair, each taking ff / ksplit of the columns
template <bool ROUND>
__global__ void __launch_bounds__(PA_DV_THREADS) pa_k_dec_expert_down(const float *__restrict__ y, const int *__restrict__ sel_e, const float *__restrict__ sel_w, int top,
                                                                      const bf16 *__restrict__ Wd, const float *__restrict__ ao, float *__restrict__ x, int dim, int ff,
                                                                      int on_input, int ksplit, float *__restrict__ dst = nullptr, const float *__restrict__ extra = nullptr,
                                                                      const float *__restrict__ extra_logit = nullptr) {
    __shared__ float part_s[8][2];
    ps_grid_dep_launch(); // the next kernel (the next layer's q|k|v rows, or the head) may start fetching its weights
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pairs = 8 / ksplit, pair = warp % pairs, slice = warp / pairs;
    const int n0 = (blockIdx.x * pairs + pair) * 2, n1 = min(n0 + 1, dim - 1);
    const int kc = ff / ksplit, k_begin = slice * kc, k_end = slice == ksplit - 1 ? ff : k_begin + kc;
    const bool live = n0 < dim;
    float t0 = 0.f, t1 = 0.f;
    if (live) {
        for (int r = 0; r < top; r++) {
            const int e = sel_e[r];
            pa_prefetch2(Wd + ((int64_t)e * dim + n0) * ff, Wd + ((int64_t)e * dim + n1) * ff, k_begin, k_end, lane);
        }
        for (int r = 0; r < top; r++) {
            const int e = sel_e[r];
            float s0, s1;
            pa_dot2<ROUND>(Wd + ((int64_t)e * dim + n0) * ff, Wd + ((int64_t)e * dim + n1) * ff, y + (int64_t)r * ff, ff, 1.0f, lane, s0, s1, k_begin, k_end);
            const float w = on_input ? 1.0f : sel_w[r];
            t0 += s0 * w;
            t1 += s1 * w;
        }
    }
    if (ksplit > 1) {
        if (lane == 0) { part_s[warp][0] = t0; part_s[warp][1] = t1; }
        __syncthreads();
        if (slice != 0) return;
        t0 = t1 = 0.f;
        for (int q = 0; q < ksplit; q++) { t0 += part_s[q * pairs + pair][0]; t1 += part_s[q * pairs + pair][1]; }
    }
    if (!live) return;
    if (dst) { // sequential blocks: the feed-forward's output waits for the next seam; a shared expert's output joins it here
        const float sg = extra ? (extra_logit ? 1.0f / (1.0f + expf(-extra_logit[0])) : 1.0f) : 0.f;
        if (lane == 0) dst[n0] = t0 + (extra ? sg * extra[n0] : 0.f);
        if (lane == 1 && n1 != n0) dst[n1] = t1 + (extra ? sg * extra[n1] : 0.f);
        return;
    }
    if (lane == 0) x[n0] += ao[n0] + t0;
    if (lane == 1 && n1 != n0) x[n1] += ao[n1] + t1;
}
