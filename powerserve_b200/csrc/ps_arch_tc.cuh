// ps_arch_tc.cuh - tcgen05 GEMM for the layer-list executor's bfloat16 products: C[token][n] = sum_k X[token][k] W[n][k].
//
// The WEIGHT rows are the MMA's M side (128 output features per unit), the tokens its N side (128 per unit), so one
// accumulator column is one token and an epilogue warp's 32 tensor-memory lanes are 32 consecutive output features: the
// stores of a column are coalesced.  Both operands reach shared memory as ready-made canonical K-major no-swizzle blocks
// ([k-chunk of 8][row][8 elements], 16 KB per 128 rows x 64 k) through ONE 1-D bulk copy each:
//   * weights are re-tiled once at bind time (pa_k_tc_tile_w), per expert for the routed feed-forward;
//   * activations are rounded to bfloat16 and tiled per call (pa_k_tc_prep_x), gathered and scaled per routed row.
// Roles per CTA (persistent over units): 4 epilogue warps, one producer lane, one MMA-issuing lane; 6 (4 for the fused
// gate|up pair) stages of 64 k; two accumulator buffers in tensor memory so the epilogue of unit i overlaps the MMAs of
// unit i + 1.  Every wait is bounded: a pipeline that loses step reports through the context's error flag.
#pragma once
#include "ps_ptx.cuh"

#define PT_M 128
#define PT_N 128
#define PT_KB 64
#define PT_BLOCK (128 * PT_KB * 2) // bytes of one operand block (either side)
#define PT_THREADS 192
#define PT_SMEM (192 * 1024 + 1024)

// ---------------------------------------------------------------------------------------------------- operand builders
// weights [groups][N][K] bf16 row-major -> blocks [group][row tile][k block][k-chunk 8][row 128][8]; zero outside N x K
__global__ void __launch_bounds__(256) pa_k_tc_tile_w(uint8_t *__restrict__ dst, const bf16 *__restrict__ w, int N, int K, int n_rt, int nkb) {
    const int kb = blockIdx.x, rt = blockIdx.y, grp = blockIdx.z;
    const bf16 *src = w + (int64_t)grp * N * K;
    uint8_t *out = dst + (((int64_t)grp * n_rt + rt) * nkb + kb) * PT_BLOCK;
    for (int c = threadIdx.x; c < 128 * 8; c += 256) {
        const int kc = c & 7, row = c >> 3, n = rt * 128 + row, k0 = kb * PT_KB + kc * 8;
        uint16_t v[8];
#pragma unroll
        for (int t = 0; t < 8; t++) v[t] = (n < N && k0 + t < K) ? reinterpret_cast<const uint16_t *>(src)[(int64_t)n * K + k0 + t] : (uint16_t)0;
        uint4 pk;
        pk.x = v[0] | ((uint32_t)v[1] << 16); pk.y = v[2] | ((uint32_t)v[3] << 16); pk.z = v[4] | ((uint32_t)v[5] << 16); pk.w = v[6] | ((uint32_t)v[7] << 16);
        *reinterpret_cast<uint4 *>(out + kc * 2048 + row * 16) = pk;
    }
}

// activations fp32 -> bf16 blocks [column tile][k block][k-chunk][token 128][8].  Dense: tile t holds rows t * 128 ..;
// routed: tile t holds rows tile_row0[t] .. tile_end[t] of the row list (token gathered through row_token, scaled by row_w).
__global__ void __launch_bounds__(256) pa_k_tc_prep_x(uint8_t *__restrict__ dst, const float *__restrict__ x, int ldx, int M, int K, int nkb, const int *__restrict__ n_tiles,
                                                      const int *__restrict__ tile_row0, const int *__restrict__ tile_end, const int *__restrict__ row_token,
                                                      const float *__restrict__ row_w) {
    const int kb = blockIdx.x, t = blockIdx.y;
    if (n_tiles && t >= *n_tiles) return;
    const int r0 = tile_row0 ? tile_row0[t] : t * 128, rend = tile_end ? tile_end[t] : M;
    uint8_t *out = dst + ((int64_t)t * nkb + kb) * PT_BLOCK;
    for (int c = threadIdx.x; c < 128 * 8; c += 256) {
        const int kc = c & 7, row = c >> 3, r = r0 + row, k0 = kb * PT_KB + kc * 8;
        uint16_t v[8];
        if (r < rend) {
            const float *src = x + (int64_t)(row_token ? row_token[r] : r) * ldx;
            const float sc = row_w ? row_w[r] : 1.0f;
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = (k0 + e < K) ? __bfloat16_as_ushort(__float2bfloat16_rn(src[k0 + e] * sc)) : (uint16_t)0;
        } else {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = 0;
        }
        uint4 pk;
        pk.x = v[0] | ((uint32_t)v[1] << 16); pk.y = v[2] | ((uint32_t)v[3] << 16); pk.z = v[4] | ((uint32_t)v[5] << 16); pk.w = v[6] | ((uint32_t)v[7] << 16);
        *reinterpret_cast<uint4 *>(out + kc * 2048 + row * 16) = pk;
    }
}

// ---------------------------------------------------------------------------------------------------- the GEMM
enum { PT_MODE_DENSE = 0, PT_MODE_EXPERT_UP = 1, PT_MODE_EXPERT_DOWN = 2 };

struct PtArgs {
    const uint8_t *a0, *a1; // weight blocks [group][row tiles][k blocks]; a1 = the second matrix of a fused pair (gate | up)
    const uint8_t *b;       // activation blocks [column tiles][k blocks]
    int nkb, n_rt, n_ct;    // n_ct: column tiles (an upper bound when n_ct_dev is given)
    const int *n_ct_dev;
    const int *tile_e, *tile_row0, *tile_end; // routed: group, first row and end row of every column tile
    int M, N;               // dense: token rows; N: output features
    int mode;
    float *C;
    int ldc;
    const float *bias;
    const int *row_token, *row_slot;
    const float *row_w;
    int top, on_input;
    PaAct act;
    int act1;               // PT_MODE_DENSE: the one-argument activation on every output (a feed-forward without a gate)
    int *err;
};

template <int NA>
__global__ void __launch_bounds__(PT_THREADS, 1) pa_k_tc_gemm(const PtArgs a) {
    constexpr int STAGES = NA == 1 ? 6 : 4;
    constexpr int STAGE_BYTES = (NA + 1) * PT_BLOCK;
    extern __shared__ __align__(1024) uint8_t pt_smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_tmem_full[2], bar_tmem_empty[2];
    __shared__ uint32_t tmem_base_smem;
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)pt_smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = a.nkb, n_ct = a.n_ct_dev ? min(*a.n_ct_dev, a.n_ct) : a.n_ct;
    const int n_units = n_ct * a.n_rt;
    const int my_units = (n_units > (int)blockIdx.x) ? (n_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { ps_mbar_init(&bar_full[s], 1); ps_mbar_init(&bar_empty[s], 1); }
        for (int b = 0; b < 2; b++) { ps_mbar_init(&bar_tmem_full[b], 1); ps_mbar_init(&bar_tmem_empty[b], 4); }
        ps_fence_barrier_init();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(ps_smem_u32(&tmem_base_smem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    ps_tc_fence_before();
    __syncthreads();
    ps_tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 4) {
        // ===== producer: one bulk copy per operand block
        if (lane == 0) {
            int g = 0;
            bool ok = true;
            for (int mu = 0; mu < my_units && ok; mu++) {
                const int u = (int)blockIdx.x + mu * (int)gridDim.x, ct = u / a.n_rt, rt = u % a.n_rt;
                const int64_t grp = a.tile_e ? a.tile_e[ct] : 0;
                const uint8_t *pa0 = a.a0 + ((grp * a.n_rt + rt) * nkb) * (int64_t)PT_BLOCK;
                const uint8_t *pa1 = NA == 2 ? a.a1 + ((grp * a.n_rt + rt) * nkb) * (int64_t)PT_BLOCK : nullptr;
                const uint8_t *pb = a.b + ((int64_t)ct * nkb) * PT_BLOCK;
                for (int kb = 0; kb < nkb; kb++, g++) {
                    const int s = g % STAGES;
                    if (g >= STAGES && !ps_tc_wait(&bar_empty[s], ((g / STAGES) - 1) & 1)) { *a.err = 1; ok = false; break; }
                    uint8_t *st = smem + (size_t)s * STAGE_BYTES;
                    ps_mbar_expect_tx(&bar_full[s], STAGE_BYTES);
                    ps_bulk_g2s(st, pa0 + (int64_t)kb * PT_BLOCK, PT_BLOCK, &bar_full[s]);
                    if (NA == 2) ps_bulk_g2s(st + PT_BLOCK, pa1 + (int64_t)kb * PT_BLOCK, PT_BLOCK, &bar_full[s]);
                    ps_bulk_g2s(st + NA * PT_BLOCK, pb + (int64_t)kb * PT_BLOCK, PT_BLOCK, &bar_full[s]);
                }
            }
        }
    } else if (warp == 5) {
        // ===== MMA issuer: kind::f16 with bfloat16 operands (a_format = b_format = 1), fp32 accumulators, K-major both
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PT_N >> 3) << 17) | ((uint32_t)(PT_M >> 4) << 24);
            int g = 0;
            bool ok = true;
            for (int mu = 0; mu < my_units && ok; mu++) {
                const int tb = mu & 1;
                if (mu >= 2 && !ps_tc_wait(&bar_tmem_empty[tb], ((mu >> 1) - 1) & 1)) { *a.err = 3; break; }
                const uint32_t td = tmem_base + tb * (NA * PT_N);
                for (int kb = 0; kb < nkb; kb++, g++) {
                    const int s = g % STAGES;
                    if (!ps_tc_wait(&bar_full[s], (g / STAGES) & 1)) { *a.err = 2; ok = false; break; }
                    ps_tc_fence_after();
                    const uint32_t sa = ps_smem_u32(smem + (size_t)s * STAGE_BYTES), sb = sa + NA * PT_BLOCK;
#pragma unroll
                    for (int j = 0; j < PT_KB / 16; j++) {
                        const uint64_t bd = ps_tc_smem_desc(sb + j * 4096, 2048, 128);
                        ps_tc_mma_f16(td, ps_tc_smem_desc(sa + j * 4096, 2048, 128), bd, idesc, (kb | j) != 0);
                        if (NA == 2) ps_tc_mma_f16(td + PT_N, ps_tc_smem_desc(sa + PT_BLOCK + j * 4096, 2048, 128), bd, idesc, (kb | j) != 0);
                    }
                    ps_tc_commit(&bar_empty[s]);
                }
                if (ok) ps_tc_commit(&bar_tmem_full[tb]);
            }
        }
    } else {
        // ===== epilogue: warp w reads tensor-memory lanes 32 w .. 32 w + 31 = 32 consecutive output features
        for (int mu = 0; mu < my_units; mu++) {
            const int u = (int)blockIdx.x + mu * (int)gridDim.x, ct = u / a.n_rt, rt = u % a.n_rt, tb = mu & 1;
            if (!ps_tc_wait(&bar_tmem_full[tb], (mu >> 1) & 1)) { *a.err = 4; break; }
            ps_tc_fence_after();
            const int n = rt * PT_M + 32 * warp + lane;
            const int r0 = a.tile_row0 ? a.tile_row0[ct] : ct * PT_N, rend = a.tile_end ? a.tile_end[ct] : a.M;
            const uint32_t t_lane = tmem_base + ((uint32_t)(32 * warp) << 16) + tb * (NA * PT_N);
            const float bias = (a.bias && n < a.N) ? a.bias[n] : 0.f;
            const int n_cols = min(PT_N, rend - r0); // warp-uniform
            for (int c0 = 0; c0 < n_cols; c0 += 16) {
                uint32_t v[16], w2[16];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                               "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                             : "r"(t_lane + c0)
                             : "memory");
                if (NA == 2)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(w2[0]), "=r"(w2[1]), "=r"(w2[2]), "=r"(w2[3]), "=r"(w2[4]), "=r"(w2[5]), "=r"(w2[6]), "=r"(w2[7]), "=r"(w2[8]), "=r"(w2[9]),
                                   "=r"(w2[10]), "=r"(w2[11]), "=r"(w2[12]), "=r"(w2[13]), "=r"(w2[14]), "=r"(w2[15])
                                 : "r"(t_lane + PT_N + c0)
                                 : "memory");
                ps_tc_ld_wait();
                if (n < a.N) {
#pragma unroll
                    for (int c = 0; c < 16; c++) {
                        const int r = r0 + c0 + c;
                        if (r >= rend) break;
                        const float acc = __uint_as_float(v[c]);
                        if (a.mode == PT_MODE_DENSE) {
                            a.C[(int64_t)r * a.ldc + n] = a.act1 ? pa_act1(acc + bias, a.act) : acc + bias;
                        } else if (a.mode == PT_MODE_EXPERT_UP) {
                            a.C[(int64_t)r * a.ldc + n] = pa_expert_act(acc, NA == 2 ? __uint_as_float(w2[c]) : 0.f, a.act);
                        } else {
                            a.C[((int64_t)a.row_token[r] * a.top + a.row_slot[r]) * a.ldc + n] = a.on_input ? acc : acc * a.row_w[r];
                        }
                    }
                }
            }
            ps_tc_fence_before();
            __syncwarp();
            if (lane == 0) ps_mbar_arrive(&bar_tmem_empty[tb]);
        }
    }
    ps_tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        ps_tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}
