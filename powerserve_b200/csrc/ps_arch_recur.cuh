// ps_arch_recur.cuh - device code of the layer-list executor's recurrent token mixers and short convolutions (ps_arch.cu).
//
// Everything here works on a batch of consecutive tokens of ONE sequence and reads the first token's position from device memory,
// so the same launches serve prompt portions and the replayed single-token step.  A sequence at position 0 starts from zero state
// whatever the state buffers hold (a cache set that is used again needs no clearing).
//
//   pa_k_short_conv      causal convolution over time on every channel, taps newest last, inputs before the batch from the `tail`
//                        (the last taps - 1 inputs of the sequence), zeros before position 0; optional bias and silu
//   pa_k_conv_tail       the tail after the batch
//   pa_k_conv_step       both for a single token
//   pa_k_qkv_whole_norm  q (all heads) and k RMS-normed as one vector each with weights; K row and V^T column into the cache
//   pa_k_rope_heads      rotate-half rotation of the first dims of every head, in place, with a scale for the heads from `h_scaled` on
//   pa_k_scan            S_t = a_t S_(t-1) + k_t (c_t v_t)^T, o_t = S_t^T q_t (+ D v_t): retention (a fixed per head, c = 1) and the
//                        state-space recurrence (a_t = exp(-exp(A_log) dt_t), c_t = dt_t, dt = softplus(raw + bias)); fp32 state,
//                        16 entries of a value column per lane in registers, tokens strictly in order (the result does not
//                        depend on how a prompt was cut)
//   pa_k_gate_gru        after an attention: the heads' outputs times their sigmoid gate, and the minGRU beside the attention
//                        (S_t = (1 - z) S_(t-1) + z cand per channel, rounds of 32 tokens, gates formed ahead of the dependent steps)
//   pa_k_gate_norm       RMS norm in equal parts around a silu gate: (y silu(g)) normed times w, or normed y times silu(g)
//   pa_k_moe_sum         sum of a token's expert slots (fixed order) plus the gated shared expert
#pragma once

__device__ __forceinline__ float pa_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float pa_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// grid (channels / 256, tokens)
__global__ void __launch_bounds__(256) pa_k_short_conv(const float *__restrict__ u, int ldu, const float *__restrict__ w, const float *__restrict__ b, int C, int T,
                                                       const float *__restrict__ tail, int act_silu, float *__restrict__ y, int ldy, const int32_t *__restrict__ pos) {
    const int t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    const int p0 = pos[0];
    float acc = b ? b[c] : 0.f;
    for (int j = 0; j < T; j++) {
        const int s = t - (T - 1) + j; // token of the batch this tap meets (negative: before the batch)
        float v = 0.f;
        if (s >= 0) v = u[(int64_t)s * ldu + c];
        else if (p0 + s >= 0) v = tail[(int64_t)(T - 1 + s) * C + c];
        acc = fmaf(w[(int64_t)c * T + j], v, acc);
    }
    y[(int64_t)t * ldy + c] = act_silu ? pa_silu(acc) : acc;
}

// a thread per channel; the tail is shifted in place oldest first (entry j takes what lay bs entries later)
__global__ void __launch_bounds__(256) pa_k_conv_tail(const float *__restrict__ u, int ldu, int C, int T, float *__restrict__ tail, const int32_t *__restrict__ pos, int bs) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    const int p0 = pos[0];
    for (int j = 0; j < T - 1; j++) {
        const int s = bs - (T - 1) + j;
        float v = 0.f;
        if (s >= 0) v = u[(int64_t)s * ldu + c];
        else if (p0 + s >= 0) v = tail[(int64_t)(T - 1 + s) * C + c];
        tail[(int64_t)j * C + c] = v;
    }
}

// single token: convolution and tail in one launch, a thread per channel (it alone touches its channel's tail)
__global__ void __launch_bounds__(256) pa_k_conv_step(const float *__restrict__ u, const float *__restrict__ w, const float *__restrict__ b, int C, int T,
                                                      float *__restrict__ tail, int act_silu, float *__restrict__ y, const int32_t *__restrict__ pos) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    const int p0 = pos[0];
    const float cur = u[c];
    float acc = b ? b[c] : 0.f;
    for (int j = 0; j < T - 1; j++) {
        const float v = p0 - (T - 1) + j >= 0 ? tail[(int64_t)j * C + c] : 0.f;
        acc = fmaf(w[(int64_t)c * T + j], v, acc);
        if (j > 0) tail[(int64_t)(j - 1) * C + c] = v;
    }
    acc = fmaf(w[(int64_t)c * T + T - 1], cur, acc);
    if (T > 1) tail[(int64_t)(T - 2) * C + c] = cur;
    y[c] = act_silu ? pa_silu(acc) : acc;
}

// one CTA per token; row = [q (qd) | k (kd) | ...], the value rows from v_off on (at the keys when the values are the un-normed keys)
__global__ void __launch_bounds__(256) pa_k_qkv_whole_norm(float *__restrict__ qkv, int ld, int qd, int kd, int vd, const float *__restrict__ wq, const float *__restrict__ wk,
                                                           float eps, float *__restrict__ kc, float *__restrict__ vct, int n_ctx, const int32_t *__restrict__ pos, int v_off) {
    __shared__ float red[8];
    const int t = blockIdx.x, p = pos[t];
    float *row = qkv + (int64_t)t * ld;
    float s = 0.f;
    for (int c = threadIdx.x; c < qd; c += 256) s = fmaf(row[c], row[c], s);
    const float iq = 1.0f / sqrtf(pa_block_sum(s, red) / (float)qd + eps);
    for (int c = threadIdx.x; c < qd; c += 256) row[c] = row[c] * iq * wq[c];
    s = 0.f;
    for (int c = threadIdx.x; c < kd; c += 256) s = fmaf(row[qd + c], row[qd + c], s);
    const float ik = 1.0f / sqrtf(pa_block_sum(s, red) / (float)kd + eps);
    for (int c = threadIdx.x; c < kd; c += 256) kc[(int64_t)p * kd + c] = row[qd + c] * ik * wk[c];
    for (int c = threadIdx.x; c < vd; c += 256) vct[(int64_t)c * n_ctx + p] = row[v_off + c];
}

// grid (entries / 256, tokens); n_heads heads of hd entries from v[t * ld] on; heads h >= h_scaled are multiplied by `scale` after the rotation
__global__ void __launch_bounds__(256) pa_k_rope_heads(float *__restrict__ v, int ld, int n_heads, int hd, PaRope rope, int h_scaled, float scale, const int32_t *__restrict__ pos) {
    const int t = blockIdx.y, p = pos[t], half = rope.dims >> 1;
    float *row = v + (int64_t)t * ld;
    for (int e = blockIdx.x * 256 + threadIdx.x; e < n_heads * hd; e += gridDim.x * 256) {
        const int hh = e / hd, c = e % hd;
        const float sc = hh >= h_scaled ? scale : 1.0f;
        float *x = row + hh * hd;
        if (c >= rope.dims) { x[c] *= sc; continue; }
        if (c >= half) continue; // written by its partner
        const double turns = (double)p * rope.freq[c];
        const float ang = (float)fma(-rint(turns * 0.15915494309189535), 6.283185307179586, turns);
        const float cs = cosf(ang) * rope.mscale, sn = sinf(ang) * rope.mscale;
        const float a = x[c], b = x[c + half];
        x[c] = (a * cs - b * sn) * sc;
        x[c + half] = (b * cs + a * sn) * sc;
    }
}

#define PA_GG_THREADS 128
#define PA_GG_TOK 32      // tokens per round of the side mixer's scan
// What follows an attention that has an output gate and / or a minGRU beside it, on the rows of the first projection
// [.. | gate (od) | z (W) | u (W) | side gate (W)]:
//   CTAs below gate_ctas (grid.y walks the tokens): att[t][c] <- att[t][c] * sigmoid(gate[t][c]) * mix_scale
//   the others (blockIdx.y = 0 only; 32 channels each), tokens strictly in order:  z = sigmoid(z_raw + bz), u = u_raw + bx,
//   cand = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), S <- (1 - z) S + z cand  (S = 0 at position 0 whatever the buffer holds),
//   att[t][od + c] = S * silu(side gate) * side_scale.
// The next product reads att rows of od + W entries against [W_o | W_side_o].
__global__ void __launch_bounds__(PA_GG_THREADS) pa_k_gate_gru(float *__restrict__ att, int ldo, const float *__restrict__ proj, int ld, int od, int g_off, float mix_scale, int gate_ctas,
                                                     int W, int z_off, const float *__restrict__ bz, const float *__restrict__ bx, float side_scale,
                                                     float *__restrict__ state, const int32_t *__restrict__ pos, int bs) {
    if ((int)blockIdx.x < gate_ctas) {
        const int c = blockIdx.x * 128 + threadIdx.x;
        if (c >= od) return;
        for (int t = blockIdx.y; t < bs; t += gridDim.y) {
            const float g = g_off >= 0 ? 1.0f / (1.0f + expf(-proj[(int64_t)t * ld + g_off + c])) : 1.0f;
            att[(int64_t)t * ldo + c] *= g * mix_scale;
        }
        return;
    }
    // 32 channels per CTA, rounds of 32 tokens: the four warps take eight tokens each, fetch their operands and form the gates side by
    // side into shared memory (nothing there depends on S); then warp 0 walks the 32 steps in order, a lane per channel - the same
    // operations per step whatever the round, so the result does not depend on how the prompt was cut
    __shared__ float za[PA_GG_TOK][32], ca[PA_GG_TOK][32], ga[PA_GG_TOK][32];
    if (blockIdx.y != 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, c = ((int)blockIdx.x - gate_ctas) * 32 + lane;
    const bool live = c < W;
    float S = (live && pos[0] > 0) ? state[c] : 0.f;
    const float b0 = live ? bz[c] : 0.f, b1 = live ? bx[c] : 0.f;
    constexpr int PER = PA_GG_TOK / (PA_GG_THREADS / 32);
    for (int t0 = 0; t0 < bs; t0 += PA_GG_TOK) {
        float zr[PER], ur[PER], gr[PER];
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int t = t0 + warp * PER + i;
            const float *row = proj + (int64_t)min(t, bs - 1) * ld + z_off;
            zr[i] = live ? row[c] : 0.f; ur[i] = live ? row[W + c] : 0.f; gr[i] = live ? row[2 * W + c] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const float u = ur[i] + b1;
            za[warp * PER + i][lane] = 1.0f / (1.0f + expf(-(zr[i] + b0)));
            ca[warp * PER + i][lane] = u >= 0.f ? u + 0.5f : 1.0f / (1.0f + expf(-u));
            ga[warp * PER + i][lane] = pa_silu(gr[i]) * side_scale;
        }
        __syncthreads();
        if (warp == 0 && live) {
            const int n = min(PA_GG_TOK, bs - t0);
#pragma unroll 8
            for (int i = 0; i < n; i++) {
                const float z = za[i][lane];
                S = (1.0f - z) * S + z * ca[i][lane];
                att[(int64_t)(t0 + i) * ldo + od + c] = S * ga[i][lane];
            }
        }
        __syncthreads();
    }
    if (warp == 0 && live) state[c] = S;
}

#define PA_SC_TOK 32    // tokens staged per round (half as many for the widest states)
#define PA_SC_WARPS 4
#define PA_SC_REGS 16   // state entries per lane
struct PaScan {
    const float *q, *k, *v;   // q[t * ldq + g * q_gs + i], k likewise (i < dk, g = the head's group), v[t * ldv + h * dv + j]
    int ldq, ldk, ldv, q_gs, k_gs;
    int H, G, dk, dv;
    const float *decay;       // [H]: a_t = decay[h], c_t = 1 (dt null)
    const float *dt;          // dt[t * lddt + h] raw step sizes: c_t = softplus(dt + dt_bias[h]), a_t = exp(-exp(a_log[h]) c_t)
    int lddt;
    const float *dt_bias, *a_log, *d_skip; // [H]; d_skip null: no skip term
    float *S;                 // [H][dv][dkp]: a value column's state entries lie together, dkp = 16 * pa_scan_il(dk)
    float *o;                 // o[t * ldo + h * dv + j]
    int ldo;
    const int32_t *pos;
    int bs;
};
// lanes that share a value column: every lane holds PA_SC_REGS state entries of it, so dk <= 16 * IL (IL a power of two, at most 16)
static inline int pa_scan_il(int dk) { int il = 1; while (il * PA_SC_REGS < dk) il *= 2; return il; }
static inline int pa_scan_dkp(int dk) { return PA_SC_REGS * pa_scan_il(dk); }
static inline int pa_scan_cols(int dk, int nc) { return 32 / pa_scan_il(dk) * PA_SC_WARPS * nc; } // value columns per CTA, nc per lane
static inline int pa_scan_tok(int dk) { return pa_scan_il(dk) <= 8 ? PA_SC_TOK : PA_SC_TOK / 2; } // tokens staged per round
static inline size_t pa_scan_smem(int dk, int nc) {
    return 4 * (size_t)pa_scan_tok(dk) * (2 * (2 * (size_t)pa_scan_dkp(dk) + pa_scan_cols(dk, nc) + 1) + pa_scan_cols(dk, nc) + 2);
}

__device__ __forceinline__ void pa_cp_async4(float *dst_smem, const float *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}

// grid (dv / columns per CTA, H).  A lane owns entries i = (m * IL + li) * 4 + e (m, e < 4) of NC columns: k and q come out of shared
// memory as float4 (lanes of a column read neighbouring float4s, lanes of different columns the same ones) and serve the lane's NC
// columns from registers; the output is reduced over the IL lanes of a column by log2(IL) shuffles, always in the same order (the
// result does not depend on NC).  The q / k / v rows (and raw step sizes) of a round of tokens arrive by asynchronous 4-byte copies
// into one of two buffers while the round before is computed.
template <int IL, int NC>
__global__ void __launch_bounds__(32 * PA_SC_WARPS) pa_k_scan(const PaScan a) {
    extern __shared__ __align__(16) float sm[];
    constexpr int CW = 32 / IL, CC = CW * PA_SC_WARPS * NC, DKP = PA_SC_REGS * IL, NT = 32 * PA_SC_WARPS, TOK = IL <= 8 ? PA_SC_TOK : PA_SC_TOK / 2;
    constexpr int BUF = TOK * (2 * DKP + CC + 1); // floats of one input buffer: q rows, k rows, v entries, raw step sizes
    const int dk = a.dk, dv = a.dv;
    float *os = sm + 2 * BUF, *as = os + TOK * CC, *cs = as + TOK;
    const int h = blockIdx.y, g = h / (a.H / a.G), j0 = blockIdx.x * CC, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int li = lane % IL, col0 = (warp * NC) * CW + lane / IL; // the lane's columns: col0 + c * CW
    const bool fresh = a.pos[0] == 0;
    float S[NC][PA_SC_REGS];
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int j = j0 + col0 + c * CW;
        const float4 *Sg = reinterpret_cast<const float4 *>(a.S + ((int64_t)h * dv + min(j, dv - 1)) * DKP) + li;
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const float4 v = (!fresh && j < dv) ? Sg[m * IL] : make_float4(0.f, 0.f, 0.f, 0.f);
            S[c][4 * m] = v.x; S[c][4 * m + 1] = v.y; S[c][4 * m + 2] = v.z; S[c][4 * m + 3] = v.w;
        }
    }
    const float rate = a.dt ? expf(a.a_log[h]) : 0.f, bias = a.dt ? a.dt_bias[h] : 0.f, fixed = a.dt ? 0.f : a.decay[h], skip = a.d_skip ? a.d_skip[h] : 0.f;
    for (int e = tid; e < 2 * BUF; e += NT) sm[e] = 0.f; // what the copies never write (entries beyond dk, columns beyond dv) stays zero
    __syncthreads();
    auto fetch = [&](int t0, int buf) {
        float *qs = sm + buf * BUF, *ks = qs + TOK * DKP, *vs = ks + TOK * DKP, *ds = vs + TOK * CC;
        const int nt = min(TOK, a.bs - t0);
        for (int tt = warp; tt < nt; tt += PA_SC_WARPS) {
            const float *qr = a.q + (int64_t)(t0 + tt) * a.ldq + g * a.q_gs, *kr = a.k + (int64_t)(t0 + tt) * a.ldk + g * a.k_gs;
            for (int i = lane; i < dk; i += 32) {
                pa_cp_async4(qs + tt * DKP + i, qr + i);
                pa_cp_async4(ks + tt * DKP + i, kr + i);
            }
            const float *vr = a.v + (int64_t)(t0 + tt) * a.ldv + h * dv + j0;
            for (int c = lane; c < CC && j0 + c < dv; c += 32) pa_cp_async4(vs + tt * CC + c, vr + c);
        }
        if (a.dt)
            for (int tt = tid; tt < nt; tt += NT) pa_cp_async4(ds + tt, a.dt + (int64_t)(t0 + tt) * a.lddt + h);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, 0);
    for (int t0 = 0, buf = 0; t0 < a.bs; t0 += TOK, buf ^= 1) {
        const int nt = min(TOK, a.bs - t0);
        const float *qs = sm + buf * BUF, *ks = qs + TOK * DKP, *vs = ks + TOK * DKP, *ds = vs + TOK * CC;
        if (t0 + TOK < a.bs) {
            fetch(t0 + TOK, buf ^ 1); // (every thread left that buffer's round behind the barrier that ended it)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        for (int tt = tid; tt < nt; tt += NT) {
            if (a.dt) {
                const float d = pa_softplus(ds[tt] + bias);
                cs[tt] = d;
                as[tt] = expf(-rate * d);
            } else {
                cs[tt] = 1.0f;
                as[tt] = fixed;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float aa = as[tt], ct = cs[tt];
            float x[NC], vv[NC], acc[NC][4];
#pragma unroll
            for (int c = 0; c < NC; c++) {
                x[c] = vs[tt * CC + col0 + c * CW];
                vv[c] = x[c] * ct;
                acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
            }
            const float4 *k4 = reinterpret_cast<const float4 *>(ks + tt * DKP) + li, *q4 = reinterpret_cast<const float4 *>(qs + tt * DKP) + li;
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const float4 kk = k4[m * IL], qq = q4[m * IL];
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    S[c][4 * m] = fmaf(aa, S[c][4 * m], kk.x * vv[c]);         acc[c][0] = fmaf(S[c][4 * m], qq.x, acc[c][0]);
                    S[c][4 * m + 1] = fmaf(aa, S[c][4 * m + 1], kk.y * vv[c]); acc[c][1] = fmaf(S[c][4 * m + 1], qq.y, acc[c][1]);
                    S[c][4 * m + 2] = fmaf(aa, S[c][4 * m + 2], kk.z * vv[c]); acc[c][2] = fmaf(S[c][4 * m + 2], qq.z, acc[c][2]);
                    S[c][4 * m + 3] = fmaf(aa, S[c][4 * m + 3], kk.w * vv[c]); acc[c][3] = fmaf(S[c][4 * m + 3], qq.w, acc[c][3]);
                }
            }
#pragma unroll
            for (int c = 0; c < NC; c++) {
                float r = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
#pragma unroll
                for (int o = IL / 2; o; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
                if (li == 0) os[tt * CC + col0 + c * CW] = fmaf(skip, x[c], r);
            }
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += PA_SC_WARPS) {
            float *orow = a.o + (int64_t)(t0 + tt) * a.ldo + h * dv + j0;
            for (int c = lane; c < CC; c += 32)
                if (j0 + c < dv) orow[c] = os[tt * CC + c];
        }
    }
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int j = j0 + col0 + c * CW;
        if (j >= dv) continue;
        float4 *Sg = reinterpret_cast<float4 *>(a.S + ((int64_t)h * dv + j) * DKP) + li;
#pragma unroll
        for (int m = 0; m < 4; m++) Sg[m * IL] = make_float4(S[c][4 * m], S[c][4 * m + 1], S[c][4 * m + 2], S[c][4 * m + 3]);
    }
}

// one CTA per (part, token); `width` entries in `parts` equal parts.  gate_first: out = N(y silu(g)) * w; else out = N(y) * silu(g) (w null: 1)
__global__ void __launch_bounds__(256) pa_k_gate_norm(const float *__restrict__ y, int ldy, const float *__restrict__ gate, int ldg, int width, int parts,
                                                      const float *__restrict__ w, int gate_first, float eps, float *__restrict__ out, int ldo) {
    __shared__ float red[8];
    const int t = blockIdx.y, ps = width / parts;
    const float *yr = y + (int64_t)t * ldy, *gr = gate + (int64_t)t * ldg;
    float *orow = out + (int64_t)t * ldo;
    {
        const int c0 = blockIdx.x * ps;
        float s = 0.f;
        for (int c = threadIdx.x; c < ps; c += 256) {
            const float v = gate_first ? yr[c0 + c] * pa_silu(gr[c0 + c]) : yr[c0 + c];
            s = fmaf(v, v, s);
        }
        const float inv = 1.0f / sqrtf(pa_block_sum(s, red) / (float)ps + eps);
        for (int c = threadIdx.x; c < ps; c += 256) {
            const float gsl = pa_silu(gr[c0 + c]), wv = w ? w[c0 + c] : 1.0f;
            orow[c0 + c] = gate_first ? yr[c0 + c] * gsl * inv * wv : yr[c0 + c] * inv * wv * gsl;
        }
    }
}

// out[t][c] = sum_r slot[t][r][c] + sgate[t] * shared[t][c]   (shared null: no shared expert; sgate null: 1)
__global__ void __launch_bounds__(256) pa_k_moe_sum(float *__restrict__ out, const float *__restrict__ slot, int top, const float *__restrict__ shared,
                                                    const float *__restrict__ sgate, int dim) {
    const int t = blockIdx.y, c = blockIdx.x * 256 + threadIdx.x;
    if (c >= dim) return;
    float y = 0.f;
    for (int r = 0; r < top; r++) y += slot[((int64_t)t * top + r) * dim + c];
    if (shared) y += (sgate ? sgate[t] : 1.0f) * shared[(int64_t)t * dim + c];
    out[(int64_t)t * dim + c] = y;
}
