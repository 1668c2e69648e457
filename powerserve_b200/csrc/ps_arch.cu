// ps_arch.cu - executor of layer-list models (include/ps_cuda.h, "layer-list models"): weights, workspace and the sm_100a
// kernels of the mechanisms a layer description can name.  The context (ps_cuda.cu) owns the stream, the cache sets and the
// public entry points; this file owns what happens between the token ids and the logits.
//
// Precision contract.  The residual stream, norms, rotation angles, attention scores / soft-max weights, router logits and the K / V
// cache are fp32 in BOTH compute modes.  PS_COMPUTE_BF16 rounds the ACTIVATION operand of every weight product to bfloat16 (weights are
// bfloat16 already) and accumulates in fp32; PS_COMPUTE_F32 feeds the fp32 activations unrounded and uses FMA chains only.
#include "ps_arch.h"

#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

typedef __nv_bfloat16 bf16;

#include "ps_arch_kernels.cuh"
#include "ps_arch_decode.cuh"
#include "ps_arch_recur.cuh"
#include "ps_arch_tc.cuh"

// ====================================================================================================================== host
struct PsArchLayer {
    ps_cuda_layer_desc d{};
    int qd = 0, kd = 0, vd = 0, od = 0; // H * qk_dim, G * qk_dim, G * v_dim, H * v_dim
    bf16 *wqkv = nullptr, *wo = nullptr, *router = nullptr, *wgate = nullptr, *wup = nullptr, *wdown = nullptr;
    float *bqkv = nullptr, *bo = nullptr, *norm = nullptr, *rel = nullptr, *mix = nullptr, *temp = nullptr;
    uint16_t *bucket = nullptr; // distance -> row of the bias table, n_ctx entries
    // tensor-core operand blocks of the matrices (bfloat16 compute only): q|k|v, o, gate, up, down (per expert)
    uint8_t *t_qkv = nullptr, *t_o = nullptr, *t_gate = nullptr, *t_up = nullptr, *t_down = nullptr;
    // sequential blocks: norm of the mixer's output, norm before the feed-forward, norm of its output
    float *norm_mix_out = nullptr, *norm_ff = nullptr, *norm_ff_out = nullptr;
    float *r1 = nullptr, *r2 = nullptr, *sink_v = nullptr, *vmix = nullptr;
    // latent attention: wqkv holds W_dq | W_dkv (pw rows); W_uq; W_uk transposed per head [H][kv_rank][qk_dim] (folded into the query);
    // W_uv per head [H][v_dim][kv_rank] (applied to the weighted sum of latents)
    int pw = 0;      // rows of the first projection (q|k|v, or q latent | kv latent | rotated key part)
    int aw = 0;      // width of the attention output rows (H * v_dim, or H * kv_rank before W_uv)
    bf16 *wuq = nullptr, *wukt = nullptr, *wuv = nullptr;
    float *dq_norm = nullptr, *dkv_norm = nullptr;
    double *rope_freq = nullptr;
    float rope_mscale = 1.0f;
    uint8_t *t_uq = nullptr;
    // generic sequential layers (raw input, recurrent mixers, short convolutions, routed experts in a sequential block)
    bool gen2 = false;
    int64_t k_floats = 0, v_floats = 0; // floats of the layer's two buffers in a cache set when they are not plain K rows / V^T rows
    float *conv_w = nullptr, *conv_b = nullptr; // short convolution [channels][taps] (attention: q | k | v channels), bias
    int conv_c = 0;                            // channels through the convolution
    float *q_norm = nullptr, *k_norm = nullptr, *decay = nullptr, *dt_bias = nullptr, *a_log = nullptr, *d_skip = nullptr, *mix_norm = nullptr;
    bf16 *wsg = nullptr, *wsu = nullptr, *wsd = nullptr; // shared expert
    uint8_t *t_sg = nullptr, *t_su = nullptr, *t_sd = nullptr;
    // values from keys, output gate, side mixer: the first projection's rows are q | k | [v] | [gate] | [z | u | side gate]; the output
    // projection reads [heads' outputs | side mixer's output] against [W_o | W_side_o] (od = its input width)
    int v_off = 0, g_off = -1, z_off = 0; // where the value rows, the gate rows and the side mixer's rows start in a projected row
    int ho = 0;                           // H * v_dim: the heads' outputs
    float *lin = nullptr, *side_b = nullptr; // distance-bias slopes [H]; side mixer's biases z | u [2 W]
    float act_a = 0.f, act_b = 0.f;       // xIELU: softplus(p), 1/2 + softplus(q)
    int n_pool = 0;                       // pooled blocks of a cache set, padded to a multiple of 4
    int64_t state_off = 0;                // the side mixer's state in the K buffer (floats from its start)
};

static inline PaAct pa_act_of(const ps_cuda_layer_desc &l) { return PaAct{l.act_limit, l.act_alpha, l.up_shift, l.act_kind}; }
static inline PaAct pa_act_of(const PsArchLayer &w) {
    return w.d.act_kind == PS_ACT_XIELU ? PaAct{0.f, w.act_a, w.act_b, PS_ACT_XIELU} : pa_act_of(w.d);
}
static inline PaRoute pa_route_of(const ps_cuda_layer_desc &l) {
    return PaRoute{l.n_experts, l.top_k, l.router_act, l.route_groups, l.route_keep, l.route_renorm, l.route_renorm_eps, l.shared_ff > 0 && l.shared_gate};
}
static inline bool pa_recurrent(const ps_cuda_layer_desc &l) { return l.mixer_kind == PS_MIXER_RETENTION || l.mixer_kind == PS_MIXER_MAMBA2; }

struct PsArch {
    ps_cuda_arch_desc d{};
    std::vector<PsArchLayer> L;
    std::vector<void *> owned;
    bool bound = false, round = true;
    bf16 *embed = nullptr, *head = nullptr;
    float *final_norm = nullptr;
    // workspace
    float *x = nullptr, *h = nullptr, *qkv = nullptr, *att = nullptr, *ao = nullptr, *S = nullptr, *logits = nullptr;
    float *y = nullptr, *slot = nullptr, *sel_w = nullptr, *row_w = nullptr;
    int *sel_e = nullptr, *row_token = nullptr, *row_slot = nullptr, *tile_e = nullptr, *tile_row0 = nullptr, *tile_end = nullptr, *n_tiles = nullptr;
    float *z = nullptr;    // router logits of the single-token step
    float *pm = nullptr, *pl = nullptr; // per-block soft-max statistics of the single-token step
    float *cq = nullptr, *lq = nullptr, *qa = nullptr, *att2 = nullptr; // latent attention: normed query latent, queries, queries with W_uk folded in, values after W_uv
    float *vsrc = nullptr; // value rows of the tokens in flight from the layer others blend theirs with
    float *x2 = nullptr;   // second residual buffer of the single-token step of sequential blocks
    float *xe = nullptr;   // the embedding output, kept for the passes of a looped model that add it back
    float *pass_steps = nullptr; // [n_pass_steps][dim]
    int pool_off = 0, stat_off = 0; // where a score row keeps its pooled scores; where the single-token step keeps their block statistics
    float *cv = nullptr, *sh = nullptr, *ffo = nullptr, *sgate = nullptr; // convolution output; shared expert's output; summed feed-forward output; shared gate per token
    int max_cv = 0, max_pool = 0;
    bool has_state = false; // some layer carries state that cannot be cut back (recurrences, convolution tails)
    int max_rq = 0, max_lq = 0, max_qa = 0, max_att2 = 0, vsrc_w = 0;
    int ldP = 0;
    int64_t ldS = 0;
    int max_qkv = 0, max_od = 0, max_h = 0, max_top = 0, max_ff = 0, max_e = 0, max_dv = 0;
    int taps_on = 0;
    std::vector<float *> taps;
    uint8_t *t_head = nullptr, *tcx = nullptr; // lm_head operand blocks; activation blocks of the current product
    int max_k = 0;
    int opt_tc = 1;     // bfloat16 batches (bs >= 2) run on the tcgen05 GEMM; 0 = the fp32-FMA tile kernels on rounded operands
    int opt_simple = 0; // 1: every batch width takes the tiled kernels (the single-token kernels are skipped; tests compare the two)
    int n_sm = 148;
    // single-token step: the experts' gate | up product needs only the router logits, so it runs beside the attention kernels
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    int opt_fork = 1;
    int opt_mv_cap = 0; // > 0: resident mat-vec CTAs per SM (0: two beside overlapping launches, four for long streams or without overlap)
    int opt_prefetch = 1; // 1: a mat-vec CTA requests its first row group into L2 before the dependency wait; 2: every next group too
    int opt_pdl = 1;    // single-token kernels on the main stream are launched with programmatic stream serialisation
    int opt_scan_nc = 0; // value columns per lane of the recurrence scan (0: chosen by the grid's size)
    bool has_seq = false, has_par = false; // some layer is a sequential / a parallel block
    bool keep_embed = false;               // some run adds the embedding output back
};

namespace {

int afail(std::string &err, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    err = buf;
    return code;
}

#define PA_CK(call)                                                                                                         \
    do {                                                                                                                    \
        cudaError_t e_ = (call);                                                                                            \
        if (e_ != cudaSuccess) return afail(err, PS_CUDA_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)
#define PA_LAUNCH()                                                                                                         \
    do {                                                                                                                    \
        if (io.n_launch) ++*io.n_launch;                                                                                    \
        cudaError_t e_ = cudaGetLastError();                                                                                \
        if (e_ != cudaSuccess) return afail(err, PS_CUDA_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

int aalloc(PsArch *a, void **p, size_t bytes, std::string &err) {
    if (bytes == 0) bytes = 16;
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) return afail(err, PS_CUDA_ERR_OOM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    a->owned.push_back(*p);
    return 0;
}

inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// a small tensor (vector / table) as fp32 on the host; bfloat16 widens exactly
int small_to_f32(const ps_cuda_tensor &t, size_t n, std::vector<float> &out, const char *what, std::string &err) {
    if (!t.host) return afail(err, PS_CUDA_ERR_INVALID, "bind: tensor %s is missing", what);
    out.resize(n);
    if (t.type == PS_TYPE_BF16) {
        const uint16_t *s = static_cast<const uint16_t *>(t.host);
        for (size_t i = 0; i < n; i++) out[i] = bf16_bits_to_f32(s[i]);
    } else if (t.type == PS_TYPE_F32) {
        memcpy(out.data(), t.host, n * 4);
    } else {
        return afail(err, PS_CUDA_ERR_UNSUPPORTED, "bind: tensor %s has type %d (bfloat16 or fp32 expected)", what, t.type);
    }
    return 0;
}

int upload_f32(PsArch *a, float **dst, const std::vector<float> &v, std::string &err) {
    int rc = aalloc(a, (void **)dst, v.size() * 4, err);
    if (rc) return rc;
    PA_CK(cudaMemcpy(*dst, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
    return 0;
}

// a bfloat16 matrix, copied into `dst` (device) as it is
int upload_mat(bf16 *dst, const ps_cuda_tensor &t, size_t n, const char *what, std::string &err) {
    if (!t.host) return afail(err, PS_CUDA_ERR_INVALID, "bind: matrix %s is missing", what);
    if (t.type != PS_TYPE_BF16) return afail(err, PS_CUDA_ERR_UNSUPPORTED, "bind: matrix %s has type %d (bfloat16 expected)", what, t.type);
    PA_CK(cudaMemcpy(dst, t.host, n * 2, cudaMemcpyHostToDevice));
    return 0;
}

// distance -> row of a bias table with `rows` rows whose last bucket starts at distance `dmax`: identity below rows / 2, then
// logarithmic.  Evaluated once on the host in float32, in the order the formula is written.
void build_bucket_table(int rows, float dmax, int n, std::vector<uint16_t> &t) {
    t.resize((size_t)n);
    const int half = rows / 2;
    const float den = (float)std::log((double)dmax / (double)half);
    for (int d = 0; d < n; d++) {
        int b;
        if (d < half) {
            b = d;
        } else {
            volatile float r = logf((float)d / (float)half);
            r = r / den;
            r = r * (float)(rows - half);
            b = std::min(rows - 1, half + (int)floorf(r));
        }
        t[(size_t)d] = (uint16_t)std::max(b, 0);
    }
}

// shared memory of the single-token kernels
size_t pa_dec_scores_smem(int H, int G, int dq) { return 4 * ((size_t)PA_DS_KEYS * (((G * dq + 3) & ~3) + 4) + (size_t)H * dq + (size_t)(PA_DS_KEYS + 1) * H + (size_t)H * H); }
// the P.V kernel splits more than 4 query heads per kv head over blockIdx.z, 4 (or fewer) to a CTA
int pa_dec_pv_split(int H, int G) { return (H / G + 3) / 4; }
int pa_dec_pv_rep(int H, int G) { const int z = pa_dec_pv_split(H, G); return (H / G + z - 1) / z; }
int pa_dec_pv_chunk(int H, int G) { return std::max(32, (PA_DP_FLOATS / (PA_DP_DIMS + pa_dec_pv_rep(H, G))) & ~31); }
size_t pa_dec_pv_smem(int H, int G) {
    const int rep = pa_dec_pv_rep(H, G);
    return 4 * ((size_t)(PA_DP_DIMS + rep) * pa_dec_pv_chunk(H, G) + (size_t)(2 + 8) * rep);
}

// a launch that may overlap the end of the kernel before it in the stream (the kernel calls griddepcontrol.wait before it reads
// anything that kernel wrote)
template <typename... KArgs, typename... Args>
cudaError_t pa_launch_dep(bool pdl, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

} // namespace

extern "C" int ps_cuda_host_rel_bucket(int distance, int rows, float max_dist) {
    if (distance < 0 || rows < 2 || !(max_dist > (float)(rows / 2))) return -1;
    std::vector<uint16_t> t;
    build_bucket_table(rows, max_dist, distance + 1, t);
    return (int)t[(size_t)distance];
}

// rotation frequencies of `dims` rotated dims, evaluated once on the host in double: base^(-2 i / dims), with factor > 0 blended
// towards f_i / factor along YaRN's ramp; returns the factor on cos / sin
static double rope_freq_host(int dims, float base, float factor, int original, float fast, float slow, double *freq) {
    const int half = dims / 2;
    double lo = 0, hi = 0, mscale = 1.0;
    if (factor > 0.f) {
        auto corr = [&](double turns) { return dims * std::log((double)original / (2.0 * M_PI * turns)) / (2.0 * std::log((double)base)); };
        lo = std::max(std::floor(corr(fast)), 0.0);
        hi = std::min(std::ceil(corr(slow)), (double)(dims - 1));
        mscale = 0.1 * std::log((double)factor) + 1.0;
    }
    for (int k = 0; k < half; k++) {
        double fr = std::pow((double)base, -2.0 * k / dims);
        if (factor > 0.f) {
            const double ramp = std::min(1.0, std::max(0.0, (k - lo) / std::max(hi - lo, 0.001)));
            fr = fr / factor * ramp + fr * (1.0 - ramp);
        }
        freq[k] = fr;
    }
    return mscale;
}
// the same table rounded to float32, for tests without a device
extern "C" float ps_cuda_host_rope_freq(int dims, float base, float factor, int original, float fast, float slow, float *freq) {
    std::vector<double> f((size_t)std::max(dims / 2, 1));
    const double m = rope_freq_host(dims, base, factor, original, fast, slow, f.data());
    for (int k = 0; k < dims / 2; k++) freq[k] = (float)f[(size_t)k];
    return (float)m;
}

int ps_arch_create(PsArch **out, const ps_cuda_arch_desc *desc, std::string &err) {
    *out = nullptr;
    const ps_cuda_arch_desc &d = *desc;
    if (d.dim <= 0 || d.vocab_size <= 0 || d.n_layers <= 0 || d.n_ctx <= 0 || d.max_batch <= 0 || !d.layers)
        return afail(err, PS_CUDA_ERR_INVALID, "layer-list descriptor has non-positive fields");
    if (d.compute != PS_COMPUTE_BF16 && d.compute != PS_COMPUTE_F32) return afail(err, PS_CUDA_ERR_INVALID, "unknown compute mode %d", d.compute);
    if (d.norm_groups < 0 || (d.norm_groups > 1 && d.dim % d.norm_groups)) return afail(err, PS_CUDA_ERR_INVALID, "width %d does not split into %d norm groups", d.dim, d.norm_groups);
    PsArch *a = new PsArch();
    a->d = d;
    a->round = d.compute == PS_COMPUTE_BF16;
    a->L.resize((size_t)d.n_layers);
    auto bail = [&](int rc) { ps_arch_destroy(a); return rc; };
    for (int i = 0; i < d.n_layers; i++) {
        const ps_cuda_layer_desc &l = d.layers[i];
        PsArchLayer &w = a->L[(size_t)i];
        w.d = l;
        (l.block_kind == PS_BLOCK_SEQUENTIAL ? a->has_seq : a->has_par) = true;
        if (l.pass_embed) a->keep_embed = true;
        if ((l.pass_embed || l.pass_step) && l.block_kind != PS_BLOCK_SEQUENTIAL) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: passes open at sequential blocks", i));
        if (l.share_weights < 0 || l.share_weights > i || l.pass_embed < 0 || l.pass_step < 0 || l.pass_step > d.n_pass_steps)
            return bail(afail(err, PS_CUDA_ERR_INVALID, "layer %d: shares the weights of run %d, pass step %d of %d", i, l.share_weights - 1, l.pass_step, d.n_pass_steps));
        if (l.share_weights > 0 && memcmp(&d.layers[l.share_weights - 1], &l, offsetof(ps_cuda_layer_desc, share_weights)) != 0)
            return bail(afail(err, PS_CUDA_ERR_INVALID, "layer %d: a run that shares weights must have the sizes of run %d", i, l.share_weights - 1));
        if (l.mixer_kind < PS_MIXER_ATTENTION || l.mixer_kind > PS_MIXER_MAMBA2) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: unknown mixer kind %d", i, l.mixer_kind));
        const bool latent = l.mixer_kind == PS_MIXER_LATENT, recur = pa_recurrent(l);
        const bool newer = l.v_is_k || l.pool > 0 || l.lin_bias || l.out_gate || l.side_kind; // mechanisms of the general sequential layer only
        w.gen2 = l.block_kind == PS_BLOCK_SEQUENTIAL && !latent &&
                 (l.raw_input || recur || l.conv_taps > 0 || l.qk_norm == PS_QKNORM_WHOLE || l.chunk > 0 || l.mlp_kind == PS_MLP_ROUTED || l.rel_buckets > 0 ||
                  l.act_kind == PS_ACT_GELU_TANH || l.shared_ff > 0 || newer);
        if (newer && (!w.gen2 || l.mixer_kind != PS_MIXER_ATTENTION))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: values from keys, pooled windows, linear distance biases, output gates and side mixers need an attention in a sequential block", i));
        if (l.v_is_k && l.v_dim != l.qk_dim) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: values from keys of size %d cannot have size %d", i, l.qk_dim, l.v_dim));
        if (l.pool < 0 || (l.pool > 0 && (l.window <= 0 || l.chunk > 0 || l.conv_taps > 0 || l.rel_buckets > 0 || l.log_bias || l.lin_bias || l.head_mix)))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: pooled blocks of %d need a window and go with no distance term, chunk, convolution or head mixing", i, l.pool));
        if ((l.side_kind != 0 && (l.side_kind != PS_MIXER_MINGRU || l.side_width <= 0 || l.conv_taps > 0)) || (l.rope_interleaved && !latent))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: side mixer %d of %d channels; interleaved rotation %d", i, l.side_kind, l.side_width, l.rope_interleaved));
        if ((l.mlp_ungated && l.mlp_kind != PS_MLP_DENSE) || (l.act_kind == PS_ACT_XIELU && !l.mlp_ungated) || (d.norm_kind == PS_NORM_LAYER && (l.block_kind != PS_BLOCK_SEQUENTIAL || l.mlp_kind == PS_MLP_ROUTED)))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: a feed-forward without a gate is dense (xIELU has no gated form); layer norms go with sequential blocks and dense feed-forwards", i));
        if (!w.gen2 && (l.raw_input || recur || l.conv_taps > 0 || l.qk_norm == PS_QKNORM_WHOLE || l.chunk > 0 || l.act_kind == PS_ACT_GELU_TANH || l.shared_ff > 0 ||
                        l.router_act == PS_ROUTER_SOFTMAX || l.route_groups > 1))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: raw sublayer inputs, recurrent mixers, convolutions, whole-projection norms, chunked masks, gelu, soft-max / grouped routers and shared experts need a sequential block", i));
        if (w.gen2 && (latent || l.v_mix || l.qk_norm == PS_QKNORM_HEAD || l.proj_bias || l.head_mix || l.head_temp))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: latent attention, value blending, per-head unit norms, projection biases and head mixing are not combined with this layer's other mechanisms", i));
        if (w.gen2 && l.mlp_kind == PS_MLP_ROUTED && !l.raw_input && d.norm_groups > 1)
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: routed experts behind a group norm", i));
        if (l.chunk < 0 || l.conv_taps < 0 || l.conv_taps > 64 || l.act_kind < PS_ACT_SWISH || l.act_kind > PS_ACT_XIELU || l.shared_ff < 0)
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: chunk %d, %d convolution taps, activation %d, shared expert of %d rows", i, l.chunk, l.conv_taps, l.act_kind, l.shared_ff));
        if (l.mixer_kind == PS_MIXER_RETENTION && (l.rope_dims < 0 || l.rope_dims > l.qk_dim || (l.rope_dims & 1) || (l.rope_dims > 0 && !(l.rope_base > 0.f)) || l.qk_dim > 256 || l.rope_factor != 0.f))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: retention with heads of %d of which %d rotate (at most 256)", i, l.qk_dim, l.rope_dims));
        if (l.mixer_kind == PS_MIXER_MAMBA2 && (l.ssm_state <= 0 || l.ssm_state > 256 || l.ssm_groups <= 0 || l.n_heads % std::max(l.ssm_groups, 1) || l.gate_norm_groups <= 0 ||
                                                (l.n_heads * l.v_dim) % std::max(l.gate_norm_groups, 1) || l.conv_taps < 1))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: state-space mixer with state %d, %d groups, %d norm parts, %d taps", i, l.ssm_state, l.ssm_groups, l.gate_norm_groups, l.conv_taps));
        if (latent && (l.q_rank <= 0 || l.kv_rank <= 0 || l.rot_dim < 0 || l.rope_dims < 0 || l.rope_dims > l.rot_dim || (l.rope_dims & 1) || (l.rope_dims > 0 && !(l.rope_base > 0.f)) ||
                       l.n_kv_heads != 1 || l.proj_bias || l.head_temp || l.head_mix || l.rel_buckets || l.qk_norm || l.v_mix || l.block_kind != PS_BLOCK_SEQUENTIAL))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: unsupported latent attention (ranks %d / %d, %d rotated dims of which %d rotate)", i, l.q_rank, l.kv_rank, l.rot_dim, l.rope_dims));
        if (l.block_kind != PS_BLOCK_PARALLEL && l.block_kind != PS_BLOCK_SEQUENTIAL) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: unknown block kind %d", i, l.block_kind));
        if (l.block_kind == PS_BLOCK_PARALLEL && (l.post_norm || l.qk_norm || l.v_mix || l.mlp_kind == PS_MLP_DENSE))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: output norms, unit-RMS q / k, value blending and the dense feed-forward need a sequential block", i));
        if (l.block_kind == PS_BLOCK_SEQUENTIAL && !w.gen2 && (l.mlp_kind == PS_MLP_ROUTED || l.proj_bias || l.head_mix || l.head_temp || l.rel_buckets))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: routed experts, projection biases, head mixing / temperatures and the bias table need a parallel block", i));
        if (l.window < 0 || l.sink < PS_SINK_NONE || l.sink > PS_SINK_LEARNED || l.v_mix < PS_VMIX_NONE || l.v_mix > PS_VMIX_BLEND)
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: window %d, sink kind %d, value blending %d", i, l.window, l.sink, l.v_mix));
        if (l.n_heads <= 0 || l.v_dim <= 0 || (!recur && l.n_heads > PA_MAX_HEADS) ||
            (l.mixer_kind != PS_MIXER_MAMBA2 && (l.qk_dim <= 0 || (!recur && (l.n_kv_heads <= 0 || l.n_heads % l.n_kv_heads)))))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: unsupported head geometry (%d / %d heads, sizes %d / %d; at most %d heads)", i, l.n_heads,
                              l.n_kv_heads, l.qk_dim, l.v_dim, PA_MAX_HEADS));
        if (l.rel_buckets < 0 || l.rel_buckets > 65535 || (l.rel_buckets > 0 && (l.rel_buckets < 2 || !(l.rel_max_dist > (float)(l.rel_buckets / 2)))))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: distance-bias table of %d rows up to distance %g", i, l.rel_buckets, (double)l.rel_max_dist));
        if (l.mlp_kind != PS_MLP_NONE && l.mlp_kind != PS_MLP_ROUTED && l.mlp_kind != PS_MLP_DENSE) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: unknown feed-forward kind %d", i, l.mlp_kind));
        if (l.mlp_kind == PS_MLP_ROUTED && (l.n_experts <= 0 || l.n_experts > PA_MAX_EXPERTS || l.top_k <= 0 || l.top_k > l.n_experts || l.expert_ff <= 0 ||
                                         (l.router_act != PS_ROUTER_SIGMOID && l.router_act != PS_ROUTER_SOFTMAX) ||
                                         (l.route_groups > 1 && (l.n_experts % l.route_groups || l.route_keep <= 0 || l.route_keep > l.route_groups || l.top_k > l.route_keep * (l.n_experts / l.route_groups)))))
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: unsupported routed feed-forward (%d experts, top %d, ff %d, router activation %d)", i, l.n_experts,
                              l.top_k, l.expert_ff, l.router_act));
        if (l.mlp_kind == PS_MLP_DENSE && l.expert_ff <= 0) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: dense feed-forward of %d rows", i, l.expert_ff));
        // the attention kernels see a latent layer as one shared key head of kv_rank + rot_dim dims whose values are the latents
        const int a_dq = latent ? l.kv_rank + l.rot_dim : l.qk_dim, a_dv = latent ? l.kv_rank : l.v_dim;
        if ((!recur && pa_dec_scores_smem(l.n_heads, l.n_kv_heads, a_dq) > 160 * 1024) || (size_t)d.dim * 4 > 160 * 1024)
            return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: %d heads of size %d (or width %d) exceed the single-token kernels' shared memory", i, l.n_heads, a_dq, d.dim));
        w.qd = l.n_heads * a_dq; w.kd = l.n_kv_heads * a_dq; w.vd = l.n_kv_heads * a_dv; w.od = l.n_heads * l.v_dim;
        w.pw = latent ? l.q_rank + l.kv_rank + l.rot_dim : w.qd + w.kd + w.vd;
        w.aw = l.n_heads * a_dv;
        w.ho = w.od;
        w.v_off = w.qd + w.kd;
        if (newer) { // q | k | [v] | [gate] | [z | u | side gate]
            w.v_off = l.v_is_k ? w.qd : w.qd + w.kd;
            w.pw = w.qd + w.kd + (l.v_is_k ? 0 : w.vd);
            if (l.out_gate) { w.g_off = w.pw; w.pw += w.ho; }
            if (l.side_kind) { w.z_off = w.pw; w.pw += 3 * l.side_width; w.od += l.side_width; w.aw = w.od; }
            int64_t kf = (int64_t)w.kd * d.n_ctx, vf = (int64_t)w.vd * d.n_ctx;
            if (l.pool > 0) {
                w.n_pool = (d.n_ctx / l.pool + 3) & ~3;
                kf += (int64_t)w.n_pool * w.kd;
                vf += (int64_t)w.n_pool * w.vd;
                a->max_pool = std::max(a->max_pool, w.n_pool);
            }
            if (l.side_kind) { w.state_off = kf; kf += l.side_width; }
            w.k_floats = kf; w.v_floats = vf;
        }
        if (l.mixer_kind == PS_MIXER_RETENTION) { // q | k | v | gate; the state S [H][v_dim][qk_dim padded] takes the place of the K rows
            w.qd = w.kd = l.n_heads * l.qk_dim; w.vd = w.od = w.aw = l.n_heads * l.v_dim;
            w.pw = 2 * w.qd + 2 * w.od;
            w.k_floats = (int64_t)l.n_heads * pa_scan_dkp(l.qk_dim) * l.v_dim; w.v_floats = 4;
        } else if (l.mixer_kind == PS_MIXER_MAMBA2) { // z | x | B | C | dt; S [H][v_dim][state padded], and the convolution's tail in the second buffer
            const int inner = l.n_heads * l.v_dim, gn = l.ssm_groups * l.ssm_state;
            w.qd = w.kd = gn; w.vd = w.od = w.aw = inner;
            w.pw = 2 * inner + 2 * gn + l.n_heads;
            w.conv_c = inner + 2 * gn;
            w.k_floats = (int64_t)l.n_heads * pa_scan_dkp(l.ssm_state) * l.v_dim; w.v_floats = std::max<int64_t>(4, (int64_t)(l.conv_taps - 1) * w.conv_c);
        } else if (w.gen2 && l.conv_taps > 0) { // the last taps - 1 projected rows follow the K rows
            w.conv_c = w.pw;
            w.k_floats = (int64_t)w.kd * d.n_ctx + (int64_t)(l.conv_taps - 1) * w.pw;
        }
        if (recur || l.conv_taps > 1 || l.side_kind) a->has_state = true;
        a->max_cv = std::max(a->max_cv, w.conv_c);
        if (l.shared_ff > 0) { a->max_ff = std::max(a->max_ff, l.shared_ff); a->max_k = std::max(a->max_k, l.shared_ff); }
        if (latent) {
            a->max_rq = std::max(a->max_rq, l.q_rank);
            a->max_lq = std::max(a->max_lq, l.n_heads * (l.qk_dim + l.rot_dim));
            a->max_qa = std::max(a->max_qa, w.qd);
            a->max_att2 = std::max(a->max_att2, w.od);
            a->max_k = std::max(a->max_k, l.q_rank);
        }
        if (l.v_mix) {
            if (a->vsrc_w && a->vsrc_w != w.vd) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d: value rows of %d entries cannot blend with rows of %d", i, w.vd, a->vsrc_w));
            if (!a->vsrc_w && l.v_mix != PS_VMIX_SOURCE) return bail(afail(err, PS_CUDA_ERR_UNSUPPORTED, "layer %d blends its values but no earlier layer supplies any", i));
            a->vsrc_w = w.vd;
        }
        a->max_qkv = std::max(a->max_qkv, w.pw);
        a->max_od = std::max(a->max_od, w.aw);
        a->max_h = std::max(a->max_h, l.n_heads);
        a->max_dv = std::max(a->max_dv, a_dv);
        a->max_k = std::max(a->max_k, std::max(d.dim, w.od));
        if (l.mlp_kind == PS_MLP_DENSE) {
            a->max_ff = std::max(a->max_ff, l.expert_ff);
            a->max_k = std::max(a->max_k, l.expert_ff);
        }
        if (l.mlp_kind == PS_MLP_ROUTED) {
            a->max_top = std::max(a->max_top, l.top_k);
            a->max_ff = std::max(a->max_ff, l.expert_ff);
            a->max_e = std::max(a->max_e, l.n_experts);
            a->max_k = std::max(a->max_k, l.expert_ff);
        }
    }
    a->d.layers = nullptr; // the caller's array need not outlive this call: the copies live in L
    const int64_t B = d.max_batch, dim = d.dim;
    if (d.norm_kind != PS_NORM_RMS && d.norm_kind != PS_NORM_LAYER) return bail(afail(err, PS_CUDA_ERR_INVALID, "unknown norm kind %d", d.norm_kind));
    a->pool_off = (d.n_ctx + 3) & ~3;
    a->ldS = (int64_t)a->pool_off + a->max_pool; // a score row: the tokens, then the pooled blocks
    int rc = 0;
    auto AL = [&](auto &ptr, size_t bytes) { if (!rc) rc = aalloc(a, (void **)&ptr, bytes, err); };
    AL(a->x, 4 * dim * B);
    AL(a->h, 4 * dim * B);
    AL(a->ao, 4 * dim * B);
    AL(a->qkv, 4 * (size_t)a->max_qkv * B);
    AL(a->att, 4 * (size_t)a->max_od * B);
    AL(a->S, 4 * (size_t)a->max_h * B * a->ldS);
    AL(a->logits, 4 * (size_t)d.vocab_size * B);
    const size_t nrow = (size_t)B * std::max(a->max_top, 1);
    AL(a->y, 4 * nrow * std::max(a->max_ff, 1));
    AL(a->slot, 4 * nrow * dim);
    AL(a->sel_w, 4 * nrow);
    AL(a->sel_e, 4 * nrow);
    AL(a->row_w, 4 * nrow);
    AL(a->row_token, 4 * nrow);
    AL(a->row_slot, 4 * nrow);
    const size_t ntile = nrow / PA_TM + (size_t)std::max(a->max_e, 1) + 1;
    if (a->round) AL(a->tcx, (nrow / PT_N + (size_t)std::max(a->max_e, 1) + 1) * (size_t)((a->max_k + PT_KB - 1) / PT_KB) * PT_BLOCK);
    AL(a->tile_e, 4 * ntile);
    AL(a->tile_row0, 4 * ntile);
    AL(a->tile_end, 4 * ntile);
    AL(a->n_tiles, 16);
    AL(a->z, 4 * ((size_t)std::max(a->max_e, 1) + 1));
    if (a->max_cv) AL(a->cv, 4 * (size_t)a->max_cv * B);
    AL(a->sh, 4 * dim * B);
    AL(a->ffo, 4 * dim * B);
    AL(a->sgate, 4 * B);
    a->stat_off = (d.n_ctx + PA_DS_KEYS - 1) / PA_DS_KEYS;
    a->ldP = a->stat_off + (a->max_pool + PA_DS_KEYS - 1) / PA_DS_KEYS;
    AL(a->xe, 4 * dim * B);
    AL(a->pm, 4 * (size_t)a->max_h * a->ldP);
    AL(a->pl, 4 * (size_t)a->max_h * a->ldP);
    AL(a->x2, 4 * dim);
    if (a->max_rq) {
        AL(a->cq, 4 * (size_t)a->max_rq * B);
        AL(a->lq, 4 * (size_t)a->max_lq * B);
        AL(a->qa, 4 * (size_t)a->max_qa * B);
        AL(a->att2, 4 * (size_t)a->max_att2 * B);
    }
    if (a->vsrc_w) AL(a->vsrc, 4 * (size_t)a->vsrc_w * B);
    if (rc) return bail(rc);
    int dev = 0;
    cudaGetDevice(&dev);
    { int v = 148; if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) a->n_sm = v; }
    if (cudaFuncSetAttribute(pa_k_dec_scores, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_dec_pv, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_dec_mv<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_dec_mv<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_dec_expert_up<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_dec_expert_up<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_dec_dense_up<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_dec_dense_up<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<8, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_scan<16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_tc_gemm<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(pa_k_tc_gemm<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_SMEM) != cudaSuccess) {
        cudaGetLastError();
        return bail(afail(err, PS_CUDA_ERR_CUDA, "cudaFuncSetAttribute(dynamic shared memory) failed"));
    }
    if (cudaStreamCreateWithFlags(&a->side, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreateWithFlags(&a->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&a->ev_join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return bail(afail(err, PS_CUDA_ERR_CUDA, "side stream / events of the single-token step could not be created"));
    }
    *out = a;
    return 0;
}

void ps_arch_destroy(PsArch *a) {
    if (!a) return;
    if (a->ev_fork) cudaEventDestroy(a->ev_fork);
    if (a->ev_join) cudaEventDestroy(a->ev_join);
    if (a->side) cudaStreamDestroy(a->side);
    for (void *p : a->owned) cudaFree(p);
    delete a;
}

size_t ps_arch_k_bytes(const PsArch *a, int layer) {
    const PsArchLayer &w = a->L[(size_t)layer];
    return 4 * (w.k_floats ? (size_t)w.k_floats : (size_t)w.kd * (size_t)a->d.n_ctx);
}
size_t ps_arch_v_bytes(const PsArch *a, int layer) {
    const PsArchLayer &w = a->L[(size_t)layer];
    return 4 * (w.v_floats ? (size_t)w.v_floats : (size_t)w.vd * (size_t)a->d.n_ctx);
}
bool ps_arch_has_state(const PsArch *a) { return a->has_state; }
float *ps_arch_logits(PsArch *a) { return a->logits; }
void ps_arch_set_taps(PsArch *a, int on) { a->taps_on = on; }
const float *ps_arch_tap(PsArch *a, int layer) { return (a->taps_on && layer >= 0 && (size_t)layer < a->taps.size()) ? a->taps[(size_t)layer] : nullptr; }
bool ps_arch_step_replayable(const PsArch *a) { return !a->opt_simple && !a->taps_on && !(a->has_seq && a->has_par); }
int ps_arch_set_option(PsArch *a, const char *name, int value) {
    if (!strcmp(name, "arch_simple")) { a->opt_simple = value; return 1; }
    if (!strcmp(name, "arch_taps")) { a->taps_on = value; return 1; }
    if (!strcmp(name, "arch_tc")) { a->opt_tc = value; return 1; }
    if (!strcmp(name, "arch_fork")) { a->opt_fork = value; return 1; }
    if (!strcmp(name, "arch_pdl")) { a->opt_pdl = value; return 1; }
    if (!strcmp(name, "arch_mv_cap")) { a->opt_mv_cap = value; return 1; }
    if (!strcmp(name, "arch_prefetch")) { a->opt_prefetch = value; return 1; }
    if (!strcmp(name, "arch_scan_nc")) { a->opt_scan_nc = value; return 1; }
    return 0;
}

int ps_arch_bind(PsArch *a, const ps_cuda_arch_weights *wt, cudaStream_t stream, std::string &err) {
    (void)stream;
    if (a->bound) return afail(err, PS_CUDA_ERR_INVALID, "bind: a model is already bound");
    const ps_cuda_arch_desc &d = a->d;
    const size_t dim = (size_t)d.dim;
    int rc;
    std::vector<float> tmp;
    auto vec = [&](float **dst, const ps_cuda_tensor &t, size_t n, const char *what, bool unit_offset) -> int {
        int r = small_to_f32(t, n, tmp, what, err);
        if (r) return r;
        if (unit_offset) for (float &v : tmp) v = 1.0f + v;
        return upload_f32(a, dst, tmp, err);
    };
    if ((rc = aalloc(a, (void **)&a->embed, 2 * dim * d.vocab_size, err)) || (rc = upload_mat(a->embed, wt->embed, dim * d.vocab_size, "embed", err))) return rc;
    if ((rc = aalloc(a, (void **)&a->head, 2 * dim * d.vocab_size, err)) || (rc = upload_mat(a->head, wt->head, dim * d.vocab_size, "head", err))) return rc;
    // a norm's weight: [dim] values, or with norm_scalar one number for all coordinates
    auto normvec = [&](float **dst, const ps_cuda_tensor &t, const char *what) -> int {
        int r = small_to_f32(t, d.norm_scalar ? 1 : dim, tmp, what, err);
        if (r) return r;
        if (d.norm_scalar) tmp.assign(dim, tmp[0]);
        if (d.norm_unit_offset) for (float &v : tmp) v = 1.0f + v;
        return upload_f32(a, dst, tmp, err);
    };
    if ((rc = normvec(&a->final_norm, wt->final_norm, "final norm"))) return rc;
    auto mat = [&](bf16 **dst, const ps_cuda_tensor &t, size_t n, const char *what) -> int {
        int r = aalloc(a, (void **)dst, 2 * n, err);
        return r ? r : upload_mat(*dst, t, n, what, err);
    };
    if (d.n_pass_steps > 0 && (rc = vec(&a->pass_steps, wt->pass_steps, (size_t)d.n_pass_steps * dim, "pass steps", false))) return rc;
    a->taps.assign((size_t)d.n_layers, nullptr);
    for (int i = 0; i < d.n_layers; i++) {
        PsArchLayer &w = a->L[(size_t)i];
        const ps_cuda_layer_desc &l = w.d;
        if (l.share_weights > 0) continue; // a repeated run: it takes the pointers of its first run below
        const ps_cuda_arch_layer_weights &s = wt->layers[i];
        char nm[64];
        snprintf(nm, sizeof nm, "layer %d", i);
        if (!l.raw_input && (rc = normvec(&w.norm, s.norm, nm))) return rc;
        const size_t nq = (size_t)w.qd, nk = (size_t)w.kd, nv = (size_t)w.vd;
        if ((rc = aalloc(a, (void **)&w.wqkv, 2 * (size_t)w.pw * dim, err))) return rc;
        if (l.mixer_kind == PS_MIXER_LATENT) {
            const size_t H = (size_t)l.n_heads, rq = (size_t)l.q_rank, rk = (size_t)l.kv_rank, dr = (size_t)l.rot_dim, dn = (size_t)l.qk_dim, dv = (size_t)l.v_dim;
            if ((rc = upload_mat(w.wqkv, s.dq, rq * dim, "dq", err)) || (rc = upload_mat(w.wqkv + rq * dim, s.dkv, (rk + dr) * dim, "dkv", err))) return rc;
            if ((rc = mat(&w.wuq, s.uq, H * (dn + dr) * rq, "uq")) || (rc = mat(&w.wuv, s.uv, H * dv * rk, "uv"))) return rc;
            if ((rc = vec(&w.dq_norm, s.dq_norm, rq, "dq norm", false)) || (rc = vec(&w.dkv_norm, s.dkv_norm, rk, "dkv norm", false))) return rc;
            // W_uk [H * dn][rk] -> per head transposed [H][rk][dn]: q_h . (W_uk,h c) = (W_uk,h^T q_h) . c
            if (!s.uk.host || s.uk.type != PS_TYPE_BF16) return afail(err, PS_CUDA_ERR_INVALID, "bind: matrix uk is missing or not bfloat16");
            std::vector<uint16_t> tr(H * rk * dn);
            const uint16_t *src = static_cast<const uint16_t *>(s.uk.host);
            for (size_t hh = 0; hh < H; hh++)
                for (size_t r = 0; r < dn; r++)
                    for (size_t c = 0; c < rk; c++) tr[(hh * rk + c) * dn + r] = src[(hh * dn + r) * rk + c];
            if ((rc = aalloc(a, (void **)&w.wukt, 2 * tr.size(), err))) return rc;
            PA_CK(cudaMemcpy(w.wukt, tr.data(), 2 * tr.size(), cudaMemcpyHostToDevice));
            if (l.rope_dims > 0) {
                std::vector<double> fd((size_t)l.rope_dims / 2);
                w.rope_mscale = (float)rope_freq_host(l.rope_dims, l.rope_base, l.rope_factor, l.rope_original, l.rope_fast, l.rope_slow, fd.data());
                if ((rc = aalloc(a, (void **)&w.rope_freq, fd.size() * 8, err))) return rc;
                PA_CK(cudaMemcpy(w.rope_freq, fd.data(), fd.size() * 8, cudaMemcpyHostToDevice));
            }
        } else if (l.mixer_kind == PS_MIXER_MAMBA2) {
            const size_t H = (size_t)l.n_heads;
            if ((rc = upload_mat(w.wqkv, s.w_in, (size_t)w.pw * dim, "in", err))) return rc;
            if ((rc = vec(&w.conv_w, s.conv_w, (size_t)w.conv_c * l.conv_taps, "convolution", false)) || (rc = vec(&w.conv_b, s.conv_b, (size_t)w.conv_c, "convolution bias", false)) ||
                (rc = vec(&w.dt_bias, s.dt_bias, H, "dt_bias", false)) || (rc = vec(&w.a_log, s.a_log, H, "A_log", false)) || (rc = vec(&w.d_skip, s.d_skip, H, "D", false)) ||
                (rc = vec(&w.mix_norm, s.mix_norm, (size_t)w.od, "mixer norm", false)))
                return rc;
        } else {
            if ((rc = upload_mat(w.wqkv, s.q, nq * dim, "q", err)) || (rc = upload_mat(w.wqkv + nq * dim, s.k, nk * dim, "k", err)) ||
                (!l.v_is_k && (rc = upload_mat(w.wqkv + (nq + nk) * dim, s.v, nv * dim, "v", err))))
                return rc;
            if (l.out_gate && (rc = upload_mat(w.wqkv + (size_t)w.g_off * dim, s.g, (size_t)w.ho * dim, "output gate", err))) return rc;
            if (l.lin_bias && (rc = vec(&w.lin, s.lin, (size_t)l.n_heads, "distance-bias slopes", false))) return rc;
            if (l.side_kind) {
                const size_t W = (size_t)l.side_width;
                if ((rc = upload_mat(w.wqkv + (size_t)w.z_off * dim, s.side_z, W * dim, "side z", err)) || (rc = upload_mat(w.wqkv + ((size_t)w.z_off + W) * dim, s.side_x, W * dim, "side x", err)) ||
                    (rc = upload_mat(w.wqkv + ((size_t)w.z_off + 2 * W) * dim, s.side_g, W * dim, "side gate", err)))
                    return rc;
                std::vector<float> b, part;
                for (const ps_cuda_tensor *t : {&s.side_z_bias, &s.side_x_bias}) {
                    if ((rc = small_to_f32(*t, W, part, "side mixer bias", err))) return rc;
                    b.insert(b.end(), part.begin(), part.end());
                }
                if ((rc = upload_f32(a, &w.side_b, b, err))) return rc;
            }
            if (l.mixer_kind == PS_MIXER_RETENTION) {
                if ((rc = upload_mat(w.wqkv + (nq + nk + nv) * dim, s.g, nv * dim, "g", err)) || (rc = vec(&w.decay, s.decay, (size_t)l.n_heads, "decay", false))) return rc;
                if (l.rope_dims > 0) {
                    std::vector<double> fd((size_t)l.rope_dims / 2);
                    rope_freq_host(l.rope_dims, l.rope_base, 0.f, 0, 0.f, 0.f, fd.data());
                    if ((rc = aalloc(a, (void **)&w.rope_freq, fd.size() * 8, err))) return rc;
                    PA_CK(cudaMemcpy(w.rope_freq, fd.data(), fd.size() * 8, cudaMemcpyHostToDevice));
                }
            }
            if (w.gen2 && l.qk_norm == PS_QKNORM_WHOLE && ((rc = vec(&w.q_norm, s.q_norm, nq, "q norm", false)) || (rc = vec(&w.k_norm, s.k_norm, nk, "k norm", false)))) return rc;
            if (w.gen2 && l.mixer_kind == PS_MIXER_ATTENTION && l.conv_taps > 0) {
                std::vector<float> cw, part;
                for (auto pr : {std::make_pair(&s.q_conv, nq), std::make_pair(&s.k_conv, nk), std::make_pair(&s.v_conv, nv)}) {
                    if ((rc = small_to_f32(*pr.first, pr.second * l.conv_taps, part, "convolution", err))) return rc;
                    cw.insert(cw.end(), part.begin(), part.end());
                }
                if ((rc = upload_f32(a, &w.conv_w, cw, err))) return rc;
            }
        }
        if ((rc = aalloc(a, (void **)&w.wo, 2 * dim * (size_t)w.od, err))) return rc;
        if (l.side_kind) { // [W_o | W_side_o]: every output row reads the heads' outputs, then the side mixer's
            const size_t ho = (size_t)w.ho, W = (size_t)l.side_width;
            if (!s.o.host || !s.side_o.host || s.o.type != PS_TYPE_BF16 || s.side_o.type != PS_TYPE_BF16) return afail(err, PS_CUDA_ERR_INVALID, "bind: matrix o or side o is missing or not bfloat16");
            std::vector<uint16_t> cat(dim * (ho + W));
            for (size_t r = 0; r < dim; r++) {
                memcpy(&cat[r * (ho + W)], static_cast<const uint16_t *>(s.o.host) + r * ho, 2 * ho);
                memcpy(&cat[r * (ho + W) + ho], static_cast<const uint16_t *>(s.side_o.host) + r * W, 2 * W);
            }
            PA_CK(cudaMemcpy(w.wo, cat.data(), 2 * cat.size(), cudaMemcpyHostToDevice));
        } else if ((rc = upload_mat(w.wo, s.o, dim * (size_t)w.od, "o", err))) {
            return rc;
        }
        if (l.block_kind == PS_BLOCK_SEQUENTIAL) {
            if (l.post_norm && (rc = normvec(&w.norm_mix_out, s.norm_mix_out, "norm of the mixer's output"))) return rc;
            if (l.mlp_kind != PS_MLP_NONE) {
                if (!l.raw_input && (rc = normvec(&w.norm_ff, s.norm_ff, "norm before the feed-forward"))) return rc;
                if (l.post_norm && (rc = normvec(&w.norm_ff_out, s.norm_ff_out, "norm of the feed-forward's output"))) return rc;
            }
        }
        if (l.log_bias && ((rc = vec(&w.r1, s.r1, (size_t)l.n_heads, "distance-bias slopes", false)) || (rc = vec(&w.r2, s.r2, (size_t)l.n_heads, "distance-bias rates", false)))) return rc;
        if (l.sink == PS_SINK_LEARNED && (rc = vec(&w.sink_v, s.sink, (size_t)l.n_heads, "sink logits", false))) return rc;
        if (l.v_mix == PS_VMIX_BLEND && (rc = vec(&w.vmix, s.vmix, 1, "value blend weight", false))) return rc;
        if (l.proj_bias) {
            std::vector<float> b, part;
            for (auto pr : {std::make_pair(&s.q_bias, nq), std::make_pair(&s.k_bias, nk), std::make_pair(&s.v_bias, nv)}) {
                if ((rc = small_to_f32(*pr.first, pr.second, part, "projection bias", err))) return rc;
                b.insert(b.end(), part.begin(), part.end());
            }
            if ((rc = upload_f32(a, &w.bqkv, b, err))) return rc;
            if ((rc = vec(&w.bo, s.o_bias, dim, "output bias", false))) return rc;
        }
        if (l.head_temp && (rc = vec(&w.temp, s.head_temp, (size_t)l.n_heads, "head temperatures", false))) return rc;
        if (l.head_mix && (rc = vec(&w.mix, s.head_mix, (size_t)l.n_heads * l.n_heads, "head mixing matrix", false))) return rc;
        if (l.rel_buckets > 0) {
            if ((rc = vec(&w.rel, s.rel, (size_t)l.rel_buckets * l.n_heads, "distance-bias table", false))) return rc;
            std::vector<uint16_t> t;
            build_bucket_table(l.rel_buckets, l.rel_max_dist, d.n_ctx, t);
            if ((rc = aalloc(a, (void **)&w.bucket, t.size() * 2, err))) return rc;
            PA_CK(cudaMemcpy(w.bucket, t.data(), t.size() * 2, cudaMemcpyHostToDevice));
        }
        if (l.mlp_kind == PS_MLP_ROUTED) {
            const size_t E = (size_t)l.n_experts, ff = (size_t)l.expert_ff;
            if (!s.gate || !s.up || !s.down) return afail(err, PS_CUDA_ERR_INVALID, "bind: layer %d has no expert tensors", i);
            const size_t sgr = (l.shared_ff > 0 && l.shared_gate) ? 1 : 0; // the shared expert's gate is one more router row
            if ((rc = aalloc(a, (void **)&w.router, 2 * (E + sgr) * dim, err)) || (rc = upload_mat(w.router, s.router, E * dim, "router", err))) return rc;
            if (sgr && (rc = upload_mat(w.router + E * dim, s.shared_sg, dim, "shared gate", err))) return rc;
            if (l.shared_ff > 0) {
                const size_t sf = (size_t)l.shared_ff;
                if ((rc = mat(&w.wsg, s.shared_gate, sf * dim, "shared gate rows")) || (rc = mat(&w.wsu, s.shared_up, sf * dim, "shared up rows")) || (rc = mat(&w.wsd, s.shared_down, sf * dim, "shared down rows"))) return rc;
            }
            if ((rc = aalloc(a, (void **)&w.wgate, 2 * E * ff * dim, err)) || (rc = aalloc(a, (void **)&w.wup, 2 * E * ff * dim, err)) ||
                (rc = aalloc(a, (void **)&w.wdown, 2 * E * ff * dim, err)))
                return rc;
            for (size_t e = 0; e < E; e++)
                if ((rc = upload_mat(w.wgate + e * ff * dim, s.gate[e], ff * dim, "expert gate", err)) ||
                    (rc = upload_mat(w.wup + e * ff * dim, s.up[e], ff * dim, "expert up", err)) ||
                    (rc = upload_mat(w.wdown + e * ff * dim, s.down[e], ff * dim, "expert down", err)))
                    return rc;
        }
        if (l.mlp_kind == PS_MLP_DENSE) {
            const size_t ff = (size_t)l.expert_ff;
            if ((!l.mlp_ungated && !s.gate) || !s.up || !s.down) return afail(err, PS_CUDA_ERR_INVALID, "bind: layer %d has no feed-forward tensors", i);
            if ((!l.mlp_ungated && (rc = mat(&w.wgate, s.gate[0], ff * dim, "gate"))) || (rc = mat(&w.wup, s.up[0], ff * dim, "up")) || (rc = mat(&w.wdown, s.down[0], ff * dim, "down"))) return rc;
            if (l.act_kind == PS_ACT_XIELU) { // the two numbers of the activation become its two factors, formed once in double
                if ((rc = small_to_f32(s.act, 2, tmp, "activation numbers", err))) return rc;
                auto softplus = [](double v) { return std::log1p(std::exp(-std::fabs(v))) + std::max(v, 0.0); };
                w.act_a = (float)softplus((double)tmp[0]);
                w.act_b = (float)(0.5 + softplus((double)tmp[1]));
            }
        }
    }
    if (a->round) {
        // tensor-core operand blocks: every matrix once more in the layout the tcgen05 GEMM streams (ps_arch_tc.cuh)
        auto tile = [&](uint8_t **dst, const bf16 *src, int groups, int N, int K) -> int {
            const int n_rt = (N + PT_M - 1) / PT_M, nkb = (K + PT_KB - 1) / PT_KB;
            int r = aalloc(a, (void **)dst, (size_t)groups * n_rt * nkb * PT_BLOCK, err);
            if (r) return r;
            pa_k_tc_tile_w<<<dim3((unsigned)nkb, (unsigned)n_rt, (unsigned)groups), 256, 0, stream>>>(*dst, src, N, K, n_rt, nkb);
            PA_CK(cudaGetLastError());
            return 0;
        };
        if ((rc = tile(&a->t_head, a->head, 1, d.vocab_size, d.dim))) return rc;
        for (int i = 0; i < d.n_layers; i++) {
            PsArchLayer &w = a->L[(size_t)i];
            if (w.d.share_weights > 0) continue;
            if ((rc = tile(&w.t_qkv, w.wqkv, 1, w.pw, d.dim)) || (rc = tile(&w.t_o, w.wo, 1, d.dim, w.od))) return rc;
            if (w.wuq && (rc = tile(&w.t_uq, w.wuq, 1, w.d.n_heads * (w.d.qk_dim + w.d.rot_dim), w.d.q_rank))) return rc;
            if (w.d.mlp_kind == PS_MLP_DENSE &&
                ((w.wgate && (rc = tile(&w.t_gate, w.wgate, 1, w.d.expert_ff, d.dim))) || (rc = tile(&w.t_up, w.wup, 1, w.d.expert_ff, d.dim)) || (rc = tile(&w.t_down, w.wdown, 1, d.dim, w.d.expert_ff))))
                return rc;
            if (w.wsg && ((rc = tile(&w.t_sg, w.wsg, 1, w.d.shared_ff, d.dim)) || (rc = tile(&w.t_su, w.wsu, 1, w.d.shared_ff, d.dim)) || (rc = tile(&w.t_sd, w.wsd, 1, d.dim, w.d.shared_ff))))
                return rc;
            if (w.d.mlp_kind == PS_MLP_ROUTED &&
                ((rc = tile(&w.t_gate, w.wgate, w.d.n_experts, w.d.expert_ff, d.dim)) || (rc = tile(&w.t_up, w.wup, w.d.n_experts, w.d.expert_ff, d.dim)) ||
                 (rc = tile(&w.t_down, w.wdown, w.d.n_experts, d.dim, w.d.expert_ff))))
                return rc;
        }
        PA_CK(cudaStreamSynchronize(stream));
    }
    for (int i = 0; i < d.n_layers; i++) { // repeated runs: the first run's weights under the run's own description
        PsArchLayer &w = a->L[(size_t)i];
        if (w.d.share_weights <= 0) continue;
        const ps_cuda_layer_desc keep = w.d;
        w = a->L[(size_t)keep.share_weights - 1];
        w.d = keep;
    }
    a->bound = true;
    return 0;
}

template <bool ROUND>
static int forward_t(PsArch *a, const PsArchIO &io, int bs, int pos0, int lm_head, std::string &err) {
    const ps_cuda_arch_desc &d = a->d;
    const int dim = d.dim, B = d.max_batch;
    const int n_kv = pos0 + bs;
    const int n_kv_cap = io.n_kv_cap > 0 ? io.n_kv_cap : n_kv; // grids of the single-token attention (a captured step covers the whole cache)
    cudaStream_t st = io.stream;
    const dim3 blk(256);
    auto cdiv = [](int64_t x, int64_t y) { return (unsigned)((x + y - 1) / y); };
    // single tokens take the single-token kernels; a model that mixes both block kinds, and taps of sequential blocks, take the batch kernels
    const bool single = bs == 1 && !a->opt_simple && !(a->has_seq && (a->has_par || a->taps_on));
    const int groups = std::max(1, d.norm_groups), center = d.norm_kind == PS_NORM_LAYER;
    // warps sharing a row pair in the single-token mat-vecs: enough CTAs to fill the GPU when the matrix has few rows
    auto pick_ksplit = [&](int rows, int K) {
        int ks = 1;
        while (ks < 8 && (rows + 16 / ks - 1) / (16 / ks) < 4 * a->n_sm && K % (16 * ks) == 0 && K / (2 * ks) >= 256) ks *= 2;
        return ks;
    };
    // the mat-vec CTAs walk the row groups with the grid's stride: at most four resident CTAs per SM, one wave
    // (two per SM when the launches overlap: the next kernel's CTAs need room beside them to fetch their weights early)
    const bool pdl = a->opt_pdl != 0;
    auto mv_grid = [&](int rows, int ks, int K) {
        // a long stream (>= 48 MB) gains more from four resident CTAs per SM than from the next kernel's early start
        const int cap = a->opt_mv_cap > 0 ? a->opt_mv_cap : (!pdl || (int64_t)rows * K * 2 >= ((int64_t)48 << 20)) ? 4 : 2;
        return std::min(cdiv(rows, PA_DV_ROWS / ks), (unsigned)(cap * a->n_sm));
    };
    const bool tc = ROUND && a->opt_tc && !single && !a->opt_simple;
    // C[m][n] = sum_k X[m][k] W[n][k] + bias[n] on the tensor cores: round + tile the activations, then the GEMM
    auto tc_dense = [&](const float *X, int ldx, int M, int K, const uint8_t *wt, int N, const float *bias, float *C, int ldc, const PaAct *act1 = nullptr) -> int {
        const int nkb = (K + PT_KB - 1) / PT_KB, n_ct = (M + PT_N - 1) / PT_N, n_rt = (N + PT_M - 1) / PT_M;
        pa_k_tc_prep_x<<<dim3((unsigned)nkb, (unsigned)n_ct), 256, 0, st>>>(a->tcx, X, ldx, M, K, nkb, nullptr, nullptr, nullptr, nullptr, nullptr);
        PA_LAUNCH();
        PtArgs g{};
        g.a0 = wt; g.b = a->tcx; g.nkb = nkb; g.n_rt = n_rt; g.n_ct = n_ct; g.M = M; g.N = N; g.mode = PT_MODE_DENSE; g.C = C; g.ldc = ldc; g.bias = bias; g.err = io.err_dev;
        if (act1) { g.act = *act1; g.act1 = 1; }
        pa_k_tc_gemm<1><<<std::min(a->n_sm, n_ct * n_rt), PT_THREADS, PT_SMEM, st>>>(g);
        PA_LAUNCH();
        return 0;
    };

    // y = X W^T for a batch: tensor cores on rounded operands, or the fp32-FMA tiles
    auto linear = [&](const float *X, int ldx, int K, const bf16 *W, const uint8_t *Wt, int N, float *Cout, int ldc) -> int {
        if (tc) return tc_dense(X, ldx, bs, K, Wt, N, nullptr, Cout, ldc);
        pa_k_linear<ROUND><<<dim3(cdiv(N, PA_TN), cdiv(bs, PA_TM)), blk, 0, st>>>(X, ldx, W, nullptr, Cout, ldc, bs, N, K, 0, 0);
        PA_LAUNCH();
        return 0;
    };
    // per-head products (blockIdx.z = head): fp32-FMA tiles in both modes
    auto linear_heads = [&](const float *X, int ldx, int x_gs, int K, const bf16 *W, int N, float *Cout, int ldc, int c_gs, int heads) -> int {
        pa_k_linear<ROUND><<<dim3(cdiv(N, PA_TN), cdiv(bs, PA_TM), (unsigned)heads), blk, 0, st>>>(X, ldx, W, nullptr, Cout, ldc, bs, N, K, x_gs, c_gs);
        PA_LAUNCH();
        return 0;
    };
    // scores -> soft-max -> P.V of a batch against the cache rows 0 .. n_kv - 1 (keys before the first query's window are skipped)
    auto attend = [&](const PaAttn &at, const float *q, int ldq, int kd, int li, int aw) -> int {
        int lo0 = at.window > 0 ? std::max(0, pos0 - at.window + 1) : 0; // the first key the first query sees
        if (at.chunk > 0) lo0 = std::max(lo0, pos0 - pos0 % at.chunk);
        const int tile0 = lo0 / PA_TN, tok_tiles = (int)cdiv(n_kv, PA_TN) - tile0;
        // pooled blocks the batch's last query sees: further key tiles behind the token tiles
        const int nv = (at.pool > 0 && n_kv - at.window >= at.pool) ? (n_kv - at.window) / at.pool : 0;
        pa_k_scores<<<dim3(tok_tiles + cdiv(nv, PA_TN), cdiv(bs, PA_TM), at.H), blk, 0, st>>>(at, q, ldq, io.kc[li], kd, a->S, io.pos_dev, bs, tile0, tok_tiles);
        PA_LAUNCH();
        pa_k_mix_softmax<<<bs, 256, 4 * (size_t)at.H * at.H, st>>>(at, a->S, io.pos_dev, bs);
        PA_LAUNCH();
        pa_k_pv<<<dim3(cdiv(at.dv, PA_TN), cdiv(bs, PA_TM), at.H), blk, 0, st>>>(at, a->S, io.vct[li], a->att, aw, io.pos_dev, bs);
        PA_LAUNCH();
        return 0;
    };
    // sequential blocks: a sublayer's output waits here until the next seam adds it (normed) to the residual stream
    const float *pend_y = nullptr, *pend_w = nullptr;
    // ... and what a new pass of a looped model adds before its first layer (the embedding output, a row of the pass steps)
    const float *add_tok = nullptr, *add_vec = nullptr;
    auto seam = [&](float *h_out, const float *w_in) -> int {
        if (!pend_y && !h_out && !add_tok && !add_vec) return 0;
        pa_k_seam_norm<<<bs, 256, 0, st>>>(a->x, pend_y, pend_w, h_out, w_in, dim, groups, d.norm_eps, center, add_tok, add_vec);
        PA_LAUNCH();
        pend_y = pend_w = add_tok = add_vec = nullptr;
        return 0;
    };
    // the single-token step of sequential blocks: the residual stream alternates between two buffers, because the CTA that stores the
    // seam's sum must not overwrite what the other CTAs of the same launch still read
    float *xc = a->x, *xo = a->x2;
    auto seam_mv = [&](PaMv &mv, const float *norm_w) {
        mv.x = xc; mv.groups = groups; mv.eps = d.norm_eps; mv.norm_w = norm_w; mv.seam_y = pend_y; mv.seam_w = pend_w;
        mv.center = center; mv.add_tok = add_tok; mv.add_vec = add_vec;
        if (pend_y || add_tok || add_vec) { mv.x_out = xo; std::swap(xc, xo); }
        pend_y = pend_w = add_tok = add_vec = nullptr;
    };
    auto dec_mv = [&](PaMv &mv, size_t smem) -> int {
        mv.ksplit = pick_ksplit(mv.N + mv.E, mv.K); mv.prefetch = a->opt_prefetch;
        pa_launch_dep(pdl, pa_k_dec_mv<ROUND>, dim3(mv_grid(mv.N + mv.E, mv.ksplit, mv.K)), dim3(PA_DV_THREADS), smem, st, mv);
        PA_LAUNCH();
        return 0;
    };
    // scores and P.V of one query against the cache; the grids do not depend on the position (a window bounds the blocks of keys)
    auto attend_single = [&](const PaAttn &at, const float *q, int li, bool pool_here = false) -> int {
        unsigned blocks = cdiv(n_kv_cap, PA_DS_KEYS);
        if (at.window > 0) blocks = std::min(blocks, cdiv(at.window, PA_DS_KEYS) + 1);
        if (at.chunk > 0) blocks = std::min(blocks, cdiv(at.chunk, PA_DS_KEYS) + 1);
        const unsigned pooled = at.pool > 0 ? cdiv(n_kv_cap / at.pool, PA_DS_KEYS) : 0; // further CTAs for the pooled blocks
        pa_launch_dep(pdl, pa_k_dec_scores, dim3(blocks + pooled), dim3(256), pa_dec_scores_smem(at.H, at.G, at.dq), st, at, q, (const float *)io.kc[li], io.pos_dev, a->S, io.err_dev, (int)blocks,
                      pool_here && pooled ? io.vct[li] : (float *)nullptr);
        PA_LAUNCH();
        pa_launch_dep(pdl, pa_k_dec_pv, dim3(cdiv(at.dv, PA_DP_DIMS), at.G, pa_dec_pv_split(at.H, at.G)), dim3(256), pa_dec_pv_smem(at.H, at.G), st, at, (const float *)a->S, (const float *)io.vct[li], io.pos_dev, a->att,
                      pa_dec_pv_chunk(at.H, at.G), io.err_dev);
        PA_LAUNCH();
        return 0;
    };
    // routed experts of a batch on the input rows X: rows grouped per expert on the device, gate | up with the activation, down into per-slot rows
    auto routed_batch = [&](const float *X, const PsArchLayer &w) -> int {
        const ps_cuda_layer_desc &l = w.d;
        const int top = l.top_k, E = l.n_experts, ff = l.expert_ff, n = bs * top;
        if (tc) {
            const int max_tiles = n / PT_N + E + 1, nkb1 = (dim + PT_KB - 1) / PT_KB, nkb2 = (ff + PT_KB - 1) / PT_KB;
            pa_k_dispatch<<<1, 256, 0, st>>>(a->sel_e, a->sel_w, n, top, E, PT_N, a->row_token, a->row_slot, a->row_w, a->tile_e, a->tile_row0, a->tile_end, a->n_tiles);
            PA_LAUNCH();
            pa_k_tc_prep_x<<<dim3((unsigned)nkb1, (unsigned)max_tiles), 256, 0, st>>>(a->tcx, X, dim, n, dim, nkb1, a->n_tiles, a->tile_row0, a->tile_end, a->row_token,
                                                                                    l.route_on_input ? a->row_w : nullptr);
            PA_LAUNCH();
            PtArgs g{};
            g.a0 = w.t_gate; g.a1 = w.t_up; g.b = a->tcx; g.nkb = nkb1; g.n_rt = (ff + PT_M - 1) / PT_M; g.n_ct = max_tiles; g.n_ct_dev = a->n_tiles;
            g.tile_e = a->tile_e; g.tile_row0 = a->tile_row0; g.tile_end = a->tile_end; g.M = n; g.N = ff; g.mode = PT_MODE_EXPERT_UP; g.C = a->y; g.ldc = ff;
            g.act = pa_act_of(l); g.err = io.err_dev;
            pa_k_tc_gemm<2><<<std::min(a->n_sm, max_tiles * g.n_rt), PT_THREADS, PT_SMEM, st>>>(g);
            PA_LAUNCH();
            pa_k_tc_prep_x<<<dim3((unsigned)nkb2, (unsigned)max_tiles), 256, 0, st>>>(a->tcx, a->y, ff, n, ff, nkb2, a->n_tiles, a->tile_row0, a->tile_end, nullptr, nullptr);
            PA_LAUNCH();
            PtArgs g2{};
            g2.a0 = w.t_down; g2.b = a->tcx; g2.nkb = nkb2; g2.n_rt = (dim + PT_M - 1) / PT_M; g2.n_ct = max_tiles; g2.n_ct_dev = a->n_tiles;
            g2.tile_e = a->tile_e; g2.tile_row0 = a->tile_row0; g2.tile_end = a->tile_end; g2.M = n; g2.N = dim; g2.mode = PT_MODE_EXPERT_DOWN; g2.C = a->slot; g2.ldc = dim;
            g2.row_token = a->row_token; g2.row_slot = a->row_slot; g2.row_w = a->row_w; g2.top = top; g2.on_input = l.route_on_input; g2.err = io.err_dev;
            pa_k_tc_gemm<1><<<std::min(a->n_sm, max_tiles * g2.n_rt), PT_THREADS, PT_SMEM, st>>>(g2);
            PA_LAUNCH();
        } else {
            const int max_tiles = n / PA_TM + E + 1;
            pa_k_dispatch<<<1, 256, 0, st>>>(a->sel_e, a->sel_w, n, top, E, PA_TM, a->row_token, a->row_slot, a->row_w, a->tile_e, a->tile_row0, a->tile_end, a->n_tiles);
            PA_LAUNCH();
            pa_k_expert_up<ROUND><<<dim3(cdiv(ff, PA_TN), max_tiles), blk, 0, st>>>(X, dim, a->row_token, a->row_w, a->tile_e, a->tile_row0, a->tile_end, a->n_tiles,
                                                                                    w.wgate, w.wup, a->y, ff, dim, l.route_on_input, pa_act_of(l));
            PA_LAUNCH();
            pa_k_expert_down<ROUND><<<dim3(cdiv(dim, PA_TN), max_tiles), blk, 0, st>>>(a->y, ff, a->row_token, a->row_slot, a->row_w, a->tile_e, a->tile_row0, a->tile_end,
                                                                                      a->n_tiles, w.wdown, a->slot, top, dim, ff, l.route_on_input);
            PA_LAUNCH();
        }
        return 0;
    };
    // the dense feed-forward of a batch: gate | up (or up alone) with the activation in the product's epilogue, then down
    auto dense_batch = [&](const float *X, const bf16 *wg, const bf16 *wu, const bf16 *wd, const uint8_t *tg, const uint8_t *tu, const uint8_t *td, int ff, const PaAct &act,
                           float *out) -> int {
        if (!wg) { // no gate
            if (tc) {
                int rc = tc_dense(X, dim, bs, dim, tu, ff, nullptr, a->y, ff, &act);
                if (rc) return rc;
            } else {
                pa_k_dense_up1<ROUND><<<dim3(cdiv(ff, PA_TN), cdiv(bs, PA_TM)), blk, 0, st>>>(X, dim, wu, a->y, bs, ff, dim, act);
                PA_LAUNCH();
            }
            return linear(a->y, ff, ff, wd, td, dim, out, dim);
        }
        if (tc) {
            const int nkb = (dim + PT_KB - 1) / PT_KB, n_ct = (bs + PT_N - 1) / PT_N;
            pa_k_tc_prep_x<<<dim3((unsigned)nkb, (unsigned)n_ct), 256, 0, st>>>(a->tcx, X, dim, bs, dim, nkb, nullptr, nullptr, nullptr, nullptr, nullptr);
            PA_LAUNCH();
            PtArgs g{};
            g.a0 = tg; g.a1 = tu; g.b = a->tcx; g.nkb = nkb; g.n_rt = (ff + PT_M - 1) / PT_M; g.n_ct = n_ct; g.M = bs; g.N = ff; g.mode = PT_MODE_EXPERT_UP;
            g.C = a->y; g.ldc = ff; g.act = act; g.err = io.err_dev;
            pa_k_tc_gemm<2><<<std::min(a->n_sm, n_ct * g.n_rt), PT_THREADS, PT_SMEM, st>>>(g);
        } else {
            pa_k_dense_up<ROUND><<<dim3(cdiv(ff, PA_TN), cdiv(bs, PA_TM)), blk, 0, st>>>(X, dim, wg, wu, a->y, bs, ff, dim, act);
        }
        PA_LAUNCH();
        return linear(a->y, ff, ff, wd, td, dim, out, dim);
    };
    // ... and of a single token: the seam in the prologue of the up rows' kernel, then the down rows; the output waits in `slot`
    auto dense_single = [&](const PsArchLayer &w, const float *w_in) -> int {
        const int ff = w.d.expert_ff;
        const unsigned rows_cta = w.wgate ? PA_DV_ROWS / 2 : PA_DV_ROWS;
        pa_launch_dep(pdl, pa_k_dec_dense_up<ROUND>, dim3(std::min(cdiv(ff, rows_cta), (unsigned)(4 * a->n_sm))), dim3(PA_DV_THREADS), 4 * (size_t)dim, st, (const float *)xc, pend_y, pend_w, w_in,
                      xo, groups, d.norm_eps, (const bf16 *)w.wgate, (const bf16 *)w.wup, a->y, ff, dim, pa_act_of(w), (const bf16 *)nullptr, 0, (float *)nullptr, center);
        PA_LAUNCH();
        std::swap(xc, xo);
        PaMv mv{};
        mv.x = a->y; mv.W = w.wdown; mv.N = dim; mv.K = ff; mv.y = a->slot;
        return dec_mv(mv, 0);
    };
    auto seq_layer = [&](int li) -> int {
        const PsArchLayer &w = a->L[(size_t)li];
        const ps_cuda_layer_desc &l = w.d;
        const int H = l.n_heads, G = l.n_kv_heads;
        const bool latent = l.mixer_kind == PS_MIXER_LATENT;
        int rc;
        if (single) {
            PaMv mv{};
            seam_mv(mv, w.norm);
            mv.W = w.wqkv; mv.N = w.pw; mv.K = dim; mv.y = a->qkv;
            if ((rc = dec_mv(mv, 4 * (size_t)dim))) return rc;
        } else {
            if ((rc = seam(a->h, w.norm))) return rc;
            if ((rc = linear(a->h, dim, dim, w.wqkv, w.t_qkv, w.pw, a->qkv, w.pw))) return rc;
        }
        PaAttn at{};
        at.H = H; at.G = G; at.scale = l.score_scale; at.sink = l.sink != PS_SINK_NONE; at.sink_v = w.sink_v; at.r1 = w.r1; at.r2 = w.r2; at.window = l.window;
        at.n_ctx = d.n_ctx; at.ldS = a->ldS; at.B = B; at.pm = a->pm; at.pl = a->pl; at.ldP = a->ldP;
        const float *q = a->qkv;
        int ldq = w.pw;
        if (latent) {
            const int rq = l.q_rank, rk = l.kv_rank, dr = l.rot_dim, dn = l.qk_dim, lqw = H * (dn + dr);
            const PaRope rope{w.rope_freq, l.rope_dims, w.rope_mscale, l.rope_interleaved};
            pa_k_latent_post<<<bs, 256, 0, st>>>(a->qkv, w.pw, rq, rk, dr, w.dq_norm, w.dkv_norm, d.norm_eps, rope, a->cq, io.kc[li], io.vct[li], d.n_ctx, io.pos_dev);
            PA_LAUNCH();
            if (single) {
                PaMv mv{};
                mv.x = a->cq; mv.W = w.wuq; mv.N = lqw; mv.K = rq; mv.y = a->lq;
                if ((rc = dec_mv(mv, 0))) return rc;
                PaMv mk{}; // W_uk folded into the query, head by head
                mk.x = a->lq; mk.W = w.wukt; mk.N = H * rk; mk.K = dn; mk.y = a->qa; mk.grp_rows = rk; mk.x_gs = dn + dr; mk.y_gs = rk + dr;
                if ((rc = dec_mv(mk, 0))) return rc;
            } else {
                if ((rc = linear(a->cq, rq, rq, w.wuq, w.t_uq, lqw, a->lq, lqw))) return rc;
                if ((rc = linear_heads(a->lq, lqw, dn + dr, dn, w.wukt, rk, a->qa, w.qd, rk + dr, H))) return rc; // W_uk folded into the query
            }
            if (dr > 0) {
                pa_k_rope_q<<<bs, 256, 0, st>>>(a->lq, a->qa, H, dn, dr, rk, rope, io.pos_dev);
                PA_LAUNCH();
            }
            at.dq = rk + dr; at.dv = rk; q = a->qa; ldq = w.qd;
        } else {
            at.dq = l.qk_dim; at.dv = l.v_dim;
            if (l.qk_norm || l.v_mix)
                pa_k_qkv_post<<<bs, 256, 0, st>>>(a->qkv, w.pw, H, G, l.qk_dim, l.v_dim, l.qk_norm, d.norm_eps, l.v_mix, w.vmix, a->vsrc, a->vsrc_w, io.kc[li], io.vct[li], d.n_ctx, io.pos_dev);
            else
                pa_k_kv_store<<<dim3(cdiv(w.kd + w.vd, 256), bs), 256, 0, st>>>(a->qkv, w.pw, w.qd, w.kd, w.vd, io.kc[li], io.vct[li], d.n_ctx, io.pos_dev, w.qd + w.kd);
            PA_LAUNCH();
        }
        if (single) {
            if ((rc = attend_single(at, q, li))) return rc;
        } else if ((rc = attend(at, q, ldq, w.kd, li, w.aw))) {
            return rc;
        }
        const float *ain = a->att;
        if (latent) { // W_uv on every head's weighted sum of latents
            if (single) {
                PaMv mv{};
                mv.x = a->att; mv.W = w.wuv; mv.N = w.od; mv.K = l.kv_rank; mv.y = a->att2; mv.grp_rows = l.v_dim; mv.x_gs = l.kv_rank; mv.y_gs = l.v_dim;
                if ((rc = dec_mv(mv, 0))) return rc;
            } else if ((rc = linear_heads(a->att, w.aw, l.kv_rank, l.kv_rank, w.wuv, l.v_dim, a->att2, w.od, l.v_dim, H))) {
                return rc;
            }
            ain = a->att2;
        }
        if (single) {
            PaMv mv{};
            mv.x = ain; mv.W = w.wo; mv.N = dim; mv.K = w.od; mv.y = a->ao;
            if ((rc = dec_mv(mv, 0))) return rc;
        } else if ((rc = linear(ain, w.od, w.od, w.wo, w.t_o, dim, a->ao, dim))) {
            return rc;
        }
        pend_y = a->ao; pend_w = l.post_norm ? w.norm_mix_out : nullptr;
        if (l.mlp_kind == PS_MLP_DENSE) {
            if (single) {
                if ((rc = dense_single(w, w.norm_ff))) return rc;
            } else {
                if ((rc = seam(a->h, w.norm_ff))) return rc;
                if ((rc = dense_batch(a->h, w.wgate, w.wup, w.wdown, w.t_gate, w.t_up, w.t_down, l.expert_ff, pa_act_of(w), a->slot))) return rc;
            }
            pend_y = a->slot; pend_w = l.post_norm ? w.norm_ff_out : nullptr;
        }
        return 0;
    };

    auto scan = [&](const PaScan &sc) -> int {
        // columns per lane: two when the grid still gives every SM a CTA (each k / q value read from shared memory then serves two columns)
        const int il = pa_scan_il(sc.dk);
        int nc = a->opt_scan_nc;
        if (nc <= 0) nc = (int64_t)cdiv(sc.dv, pa_scan_cols(sc.dk, 2)) * sc.H >= (bs > 1 ? a->n_sm * 3 / 4 : 4 * a->n_sm) ? 2 : 1;
        const dim3 grid(cdiv(sc.dv, pa_scan_cols(sc.dk, nc)), (unsigned)sc.H), blk_s(32 * PA_SC_WARPS);
        const size_t smem = pa_scan_smem(sc.dk, nc);
#define PA_SCAN_CASE(IL_)                                                              \
    case IL_:                                                                           \
        if (nc == 2) pa_k_scan<IL_, 2><<<grid, blk_s, smem, st>>>(sc);                  \
        else pa_k_scan<IL_, 1><<<grid, blk_s, smem, st>>>(sc);                          \
        break;
        switch (il) {
            PA_SCAN_CASE(1) PA_SCAN_CASE(2) PA_SCAN_CASE(4) PA_SCAN_CASE(8)
        default:
            if (nc == 2) pa_k_scan<16, 2><<<grid, blk_s, smem, st>>>(sc);
            else pa_k_scan<16, 1><<<grid, blk_s, smem, st>>>(sc);
            break;
        }
#undef PA_SCAN_CASE
        PA_LAUNCH();
        return 0;
    };
    // A sequential block from the general parts: the sublayers read the residual stream itself (raw_input) or its norm; the mixer is an
    // attention (optional short convolutions, whole-projection norms, distance-bias table, window / chunks), a retention or a
    // state-space recurrence; the feed-forward is dense or routed (with an optional shared expert).  Every sublayer's output waits
    // for the next seam.  Single tokens take the weight-streaming mat-vecs with the seam in their prologues; the small kernels
    // between them are the batch's own (they read the position from device memory).
    auto gen_layer = [&](int li) -> int {
        const PsArchLayer &w = a->L[(size_t)li];
        const ps_cuda_layer_desc &l = w.d;
        const int H = l.n_heads;
        const bool raw = l.raw_input != 0;
        int rc;
        // single token, attention without convolution or q / k norm: the K rows (and V rows) go from the mat-vec straight into the cache
        const bool direct = single && l.mixer_kind == PS_MIXER_ATTENTION && l.conv_taps == 0 && l.qk_norm == PS_QKNORM_NONE;
        if (single) {
            PaMv mv{};
            seam_mv(mv, raw ? nullptr : w.norm);
            mv.W = w.wqkv; mv.N = w.pw; mv.K = dim; mv.y = a->qkv;
            if (direct) {
                mv.qd = w.qd; mv.kd = w.kd; mv.vd = l.v_is_k ? 0 : w.vd; mv.v_is_k = l.v_is_k; mv.kc = io.kc[li]; mv.vct = io.vct[li]; mv.n_ctx = d.n_ctx; mv.pos = io.pos_dev;
            }
            if ((rc = dec_mv(mv, 4 * (size_t)dim))) return rc;
        } else {
            if ((rc = seam(raw ? nullptr : a->h, raw ? nullptr : w.norm))) return rc;
            if ((rc = linear(raw ? a->x : a->h, dim, dim, w.wqkv, w.t_qkv, w.pw, a->qkv, w.pw))) return rc;
        }
        if (l.mixer_kind == PS_MIXER_ATTENTION) {
            float *q = a->qkv;
            if (l.conv_taps > 0) {
                float *tail = io.kc[li] + (int64_t)w.kd * d.n_ctx;
                if (bs == 1) {
                    pa_k_conv_step<<<cdiv(w.pw, 256), 256, 0, st>>>(a->qkv, w.conv_w, nullptr, w.pw, l.conv_taps, tail, 0, a->cv, io.pos_dev);
                } else {
                    pa_k_short_conv<<<dim3(cdiv(w.pw, 256), bs), 256, 0, st>>>(a->qkv, w.pw, w.conv_w, nullptr, w.pw, l.conv_taps, tail, 0, a->cv, w.pw, io.pos_dev);
                    if (l.conv_taps > 1) {
                        PA_LAUNCH();
                        pa_k_conv_tail<<<cdiv(w.pw, 256), 256, 0, st>>>(a->qkv, w.pw, w.pw, l.conv_taps, tail, io.pos_dev, bs);
                    }
                }
                PA_LAUNCH();
                q = a->cv;
            }
            if (l.qk_norm == PS_QKNORM_WHOLE) {
                pa_k_qkv_whole_norm<<<bs, 256, 0, st>>>(q, w.pw, w.qd, w.kd, w.vd, w.q_norm, w.k_norm, d.norm_eps, io.kc[li], io.vct[li], d.n_ctx, io.pos_dev, w.v_off);
                PA_LAUNCH();
            } else if (!direct) {
                pa_k_kv_store<<<dim3(cdiv(w.kd + w.vd, 256), bs), 256, 0, st>>>(q, w.pw, w.qd, w.kd, w.vd, io.kc[li], io.vct[li], d.n_ctx, io.pos_dev, w.v_off);
                PA_LAUNCH();
            }
            if (l.pool > 0 && !single) { // the means of the blocks that this batch completes (at most bs / pool + 1 of them); a single token's scores kernel forms its own
                pa_k_pool_blocks<<<dim3(cdiv(w.kd + w.vd, 256), (unsigned)(bs / l.pool + 1)), 256, 0, st>>>(io.kc[li], io.vct[li], w.kd, w.vd, d.n_ctx, l.pool, w.n_pool, io.pos_dev, bs);
                PA_LAUNCH();
            }
            PaAttn at{};
            at.H = H; at.G = l.n_kv_heads; at.dq = l.qk_dim; at.dv = l.v_dim; at.scale = l.score_scale; at.rel = w.rel; at.bucket = w.bucket; at.n_bucket = d.n_ctx;
            at.sink = l.sink != PS_SINK_NONE; at.sink_v = w.sink_v; at.r1 = w.r1; at.r2 = w.r2; at.window = l.window; at.chunk = l.chunk;
            at.n_ctx = d.n_ctx; at.ldS = a->ldS; at.B = B; at.pm = a->pm; at.pl = a->pl; at.ldP = a->ldP;
            at.lin = w.lin; at.pool = l.pool; at.n_pool = w.n_pool; at.pool_off = a->pool_off; at.stat_off = a->stat_off;
            if (single) rc = attend_single(at, q, li, true);
            else rc = attend(at, q, w.pw, w.kd, li, w.aw);
            if (rc) return rc;
            if (l.out_gate || l.side_kind) { // the heads' outputs through their gate; the side mixer's recurrence fills the columns behind them
                const unsigned gate_ctas = cdiv(w.ho, PA_GG_THREADS), side_ctas = l.side_kind ? cdiv(l.side_width, 32) : 0;
                pa_k_gate_gru<<<dim3(gate_ctas + side_ctas, (unsigned)std::min(bs, 64)), PA_GG_THREADS, 0, st>>>(a->att, w.aw, a->qkv, w.pw, w.ho, l.out_gate ? w.g_off : -1, l.side_kind ? l.mix_scale : 1.0f,
                                                                                                     (int)gate_ctas, l.side_kind ? l.side_width : 0, w.z_off, w.side_b, l.side_kind ? w.side_b + l.side_width : nullptr,
                                                                                                     l.side_scale, io.kc[li] + w.state_off, io.pos_dev, bs);
                PA_LAUNCH();
            }
        } else if (l.mixer_kind == PS_MIXER_RETENTION) {
            const int dq = l.qk_dim, dv = l.v_dim;
            const PaRope rope{w.rope_freq, l.rope_dims, 1.0f, 0};
            pa_k_rope_heads<<<dim3(cdiv(2 * H * dq, 256), bs), 256, 0, st>>>(a->qkv, w.pw, 2 * H, dq, rope, H, 1.0f / sqrtf((float)dq), io.pos_dev); // q | k rotated, k scaled
            PA_LAUNCH();
            PaScan sc{};
            sc.q = a->qkv; sc.k = a->qkv + w.qd; sc.v = a->qkv + 2 * w.qd; sc.ldq = sc.ldk = sc.ldv = w.pw; sc.q_gs = sc.k_gs = dq;
            sc.H = sc.G = H; sc.dk = dq; sc.dv = dv; sc.decay = w.decay; sc.S = io.kc[li]; sc.o = a->att; sc.ldo = w.od; sc.pos = io.pos_dev; sc.bs = bs;
            if ((rc = scan(sc))) return rc;
            pa_k_gate_norm<<<dim3((unsigned)H, bs), 256, 0, st>>>(a->att, w.od, a->qkv + 2 * w.qd + w.od, w.pw, w.od, H, nullptr, 0, d.norm_eps, a->att, w.od);
            PA_LAUNCH();
        } else { // PS_MIXER_MAMBA2
            const int inner = w.od, gn = l.ssm_groups * l.ssm_state, T = std::max(1, l.conv_taps);
            float *tail = io.vct[li];
            if (bs == 1) {
                pa_k_conv_step<<<cdiv(w.conv_c, 256), 256, 0, st>>>(a->qkv + inner, w.conv_w, w.conv_b, w.conv_c, T, tail, 1, a->cv, io.pos_dev);
                PA_LAUNCH();
            } else {
                pa_k_short_conv<<<dim3(cdiv(w.conv_c, 256), bs), 256, 0, st>>>(a->qkv + inner, w.pw, w.conv_w, w.conv_b, w.conv_c, T, tail, 1, a->cv, w.conv_c, io.pos_dev);
                PA_LAUNCH();
                if (T > 1) {
                    pa_k_conv_tail<<<cdiv(w.conv_c, 256), 256, 0, st>>>(a->qkv + inner, w.pw, w.conv_c, T, tail, io.pos_dev, bs);
                    PA_LAUNCH();
                }
            }
            PaScan sc{};
            sc.q = a->cv + inner + gn; sc.k = a->cv + inner; sc.v = a->cv; sc.ldq = sc.ldk = sc.ldv = w.conv_c; sc.q_gs = sc.k_gs = l.ssm_state;
            sc.H = H; sc.G = l.ssm_groups; sc.dk = l.ssm_state; sc.dv = l.v_dim; sc.dt = a->qkv + 2 * inner + 2 * gn; sc.lddt = w.pw;
            sc.dt_bias = w.dt_bias; sc.a_log = w.a_log; sc.d_skip = w.d_skip; sc.S = io.kc[li]; sc.o = a->att; sc.ldo = inner; sc.pos = io.pos_dev; sc.bs = bs;
            if ((rc = scan(sc))) return rc;
            pa_k_gate_norm<<<dim3((unsigned)l.gate_norm_groups, bs), 256, 0, st>>>(a->att, inner, a->qkv, w.pw, inner, l.gate_norm_groups, w.mix_norm, 1, d.norm_eps, a->att, inner);
            PA_LAUNCH();
        }
        if (single) {
            PaMv mv{};
            mv.x = a->att; mv.W = w.wo; mv.N = dim; mv.K = w.od; mv.y = a->ao;
            if ((rc = dec_mv(mv, 0))) return rc;
        } else if ((rc = linear(a->att, w.od, w.od, w.wo, w.t_o, dim, a->ao, dim))) {
            return rc;
        }
        pend_y = a->ao; pend_w = l.post_norm ? w.norm_mix_out : nullptr;
        if (l.mlp_kind == PS_MLP_NONE) return 0;
        const float *w_in = raw ? nullptr : w.norm_ff;
        const PaAct act = pa_act_of(w);
        const unsigned up_cap = (unsigned)(4 * a->n_sm);
        if (l.mlp_kind == PS_MLP_DENSE) {
            const int ff = l.expert_ff;
            if (single) {
                if ((rc = dense_single(w, w_in))) return rc;
            } else {
                if ((rc = seam(raw ? nullptr : a->h, w_in))) return rc;
                if ((rc = dense_batch(raw ? a->x : a->h, w.wgate, w.wup, w.wdown, w.t_gate, w.t_up, w.t_down, ff, act, a->slot))) return rc;
            }
            pend_y = a->slot; pend_w = l.post_norm ? w.norm_ff_out : nullptr;
            return 0;
        }
        // routed experts (+ shared expert)
        const int E = l.n_experts, ff = l.expert_ff, top = l.top_k, sff = l.shared_ff;
        const PaRoute rt = pa_route_of(l);
        if (single) {
            const int n_rt = E + (rt.shared_gate ? 1 : 0); // the router's rows (+ the shared gate's): logits from the unrounded input
            if (sff > 0) { // the shared expert's gate | up launch carries the seam and the router's rows
                pa_launch_dep(pdl, pa_k_dec_dense_up<ROUND>, dim3(std::min(cdiv(sff + n_rt, PA_DV_ROWS / 2), up_cap)), dim3(PA_DV_THREADS), 4 * (size_t)dim, st, (const float *)xc, pend_y, pend_w, w_in,
                              xo, groups, d.norm_eps, (const bf16 *)w.wsg, (const bf16 *)w.wsu, a->y, sff, dim, act, (const bf16 *)w.router, n_rt, a->z, 0);
                PA_LAUNCH();
                std::swap(xc, xo);
                pend_y = pend_w = nullptr;
                PaMv ms{};
                ms.x = a->y; ms.W = w.wsd; ms.N = dim; ms.K = sff; ms.y = a->sh;
                if ((rc = dec_mv(ms, 0))) return rc;
            } else {
                PaMv mv{};
                seam_mv(mv, w_in);
                mv.W = nullptr; mv.N = 0; mv.K = dim; mv.Wr = w.router; mv.E = n_rt; mv.z = a->z;
                if ((rc = dec_mv(mv, 4 * (size_t)dim))) return rc;
            }
            pa_k_dec_expert_up<ROUND><<<dim3(std::min(cdiv(ff, PA_DV_ROWS / 2), (unsigned)std::max(1, 4 * a->n_sm / top)), top), PA_DV_THREADS, 4 * (size_t)dim, st>>>(
                xc, w_in, d.norm_eps, a->z, rt, w.wgate, w.wup, a->y, ff, dim, l.route_on_input, act, a->sel_e, a->sel_w);
            PA_LAUNCH();
            const int ksd = pick_ksplit(dim, ff);
            pa_k_dec_expert_down<ROUND><<<cdiv(dim, PA_DV_ROWS / ksd), PA_DV_THREADS, 0, st>>>(a->y, a->sel_e, a->sel_w, top, w.wdown, nullptr, nullptr, dim, ff, l.route_on_input, ksd, a->ffo,
                                                                                               sff > 0 ? a->sh : nullptr, rt.shared_gate ? a->z + E : nullptr);
            PA_LAUNCH();
        } else {
            if ((rc = seam(raw ? nullptr : a->h, w_in))) return rc;
            const float *X = raw ? a->x : a->h;
            if (sff > 0 && (rc = dense_batch(X, w.wsg, w.wsu, w.wsd, w.t_sg, w.t_su, w.t_sd, sff, act, a->sh))) return rc;
            pa_k_router<<<bs, 256, 0, st>>>(X, w.router, dim, rt, a->sel_e, a->sel_w, a->sgate);
            PA_LAUNCH();
            if ((rc = routed_batch(X, w))) return rc;
            pa_k_moe_sum<<<dim3(cdiv(dim, 256), bs), 256, 0, st>>>(a->ffo, a->slot, top, sff > 0 ? a->sh : nullptr, rt.shared_gate ? a->sgate : nullptr, dim);
            PA_LAUNCH();
        }
        pend_y = a->ffo; pend_w = l.post_norm ? w.norm_ff_out : nullptr;
        return 0;
    };

    pa_k_embed<<<bs, 128, 0, st>>>(a->x, a->embed, io.tokens_dev, dim, d.embed_scale, a->keep_embed ? a->xe : nullptr);
    PA_LAUNCH();
    for (int li = 0; li < d.n_layers; li++) {
        const PsArchLayer &w = a->L[(size_t)li];
        const ps_cuda_layer_desc &l = w.d;
        if (l.pass_embed) add_tok = a->xe;   // a new pass: the run's first seam adds these to the stream
        if (l.pass_step) add_vec = a->pass_steps + (int64_t)(l.pass_step - 1) * dim;
        if (l.block_kind == PS_BLOCK_SEQUENTIAL) {
            int rc = w.gen2 ? gen_layer(li) : seq_layer(li);
            if (rc) return rc;
            if (a->taps_on) {
                if ((rc = seam(nullptr, nullptr))) return rc; // the tap shows the layer's whole effect
                if (!a->taps[(size_t)li]) { rc = aalloc(a, (void **)&a->taps[(size_t)li], 4 * (size_t)dim * B, err); if (rc) return rc; }
                PA_CK(cudaMemcpyAsync(a->taps[(size_t)li], a->x, 4 * (size_t)dim * bs, cudaMemcpyDeviceToDevice, st));
            }
            continue;
        }
        if (pend_y) { int rc = seam(nullptr, nullptr); if (rc) return rc; }
        const int H = l.n_heads, G = l.n_kv_heads, dq = l.qk_dim, dv = l.v_dim, nqkv = w.qd + w.kd + w.vd;
        const bool routed = l.mlp_kind == PS_MLP_ROUTED;
        if (!single) { // (the single-token kernels norm in their prologues)
            pa_k_norm<<<bs, 256, 0, st>>>(a->h, a->x, w.norm, dim, d.norm_eps);
            PA_LAUNCH();
        }
        // ---- token mixer: projections -> cache -> scores -> (mix, soft-max) -> P.V -> output projection
        if (single) {
            PaMv mv{};
            mv.x = a->x; mv.norm_w = w.norm; mv.eps = d.norm_eps; mv.W = w.wqkv; mv.bias = w.bqkv; mv.N = nqkv; mv.K = dim; mv.y = a->qkv;
            mv.qd = w.qd; mv.kd = w.kd; mv.vd = w.vd; mv.kc = io.kc[li]; mv.vct = io.vct[li]; mv.n_ctx = d.n_ctx; mv.pos = io.pos_dev;
            if (routed) { mv.Wr = w.router; mv.E = l.n_experts; mv.z = a->z; }
            mv.ksplit = pick_ksplit(nqkv + mv.E, dim); mv.prefetch = a->opt_prefetch;
            pa_launch_dep(pdl, pa_k_dec_mv<ROUND>, dim3(mv_grid(nqkv + mv.E, mv.ksplit, dim)), dim3(PA_DV_THREADS), 4 * (size_t)dim, st, mv);
            if (routed) {
                // gate | up of the chosen experts: reads x and the router logits only, so it runs on the side stream while the main
                // stream goes through scores, P.V and the output projection (a fork in the captured graph); joined before `down`
                PA_LAUNCH();
                cudaStream_t se = a->opt_fork ? a->side : st;
                if (a->opt_fork) { PA_CK(cudaEventRecord(a->ev_fork, st)); PA_CK(cudaStreamWaitEvent(se, a->ev_fork, 0)); }
                pa_k_dec_expert_up<ROUND><<<dim3(std::min(cdiv(l.expert_ff, PA_DV_ROWS / 2), (unsigned)std::max(1, 4 * a->n_sm / l.top_k)), l.top_k), PA_DV_THREADS, 4 * (size_t)dim, se>>>(
                    a->x, w.norm, d.norm_eps, a->z, pa_route_of(l), w.wgate, w.wup, a->y, l.expert_ff, dim, l.route_on_input, pa_act_of(l),
                    a->sel_e, a->sel_w);
                if (a->opt_fork) PA_CK(cudaEventRecord(a->ev_join, se));
            }
        } else if (tc) {
            int rc = tc_dense(a->h, dim, bs, dim, w.t_qkv, nqkv, w.bqkv, a->qkv, nqkv);
            if (rc) return rc;
        } else {
            pa_k_linear<ROUND><<<dim3(cdiv(nqkv, PA_TN), cdiv(bs, PA_TM)), blk, 0, st>>>(a->h, dim, w.wqkv, w.bqkv, a->qkv, nqkv, bs, nqkv, dim);
        }
        PA_LAUNCH();
        if (!single) {
            pa_k_kv_store<<<dim3(cdiv(w.kd + w.vd, 256), bs), 256, 0, st>>>(a->qkv, nqkv, w.qd, w.kd, w.vd, io.kc[li], io.vct[li], d.n_ctx, io.pos_dev, w.qd + w.kd);
            PA_LAUNCH();
        }
        PaAttn at{};
        at.sink_v = w.sink_v; at.r1 = w.r1; at.r2 = w.r2; at.window = l.window;
        at.H = H; at.G = G; at.dq = dq; at.dv = dv; at.scale = l.score_scale; at.temp = w.temp; at.rel = w.rel; at.bucket = w.bucket; at.n_bucket = d.n_ctx;
        at.mix = w.mix; at.sink = l.sink != PS_SINK_NONE; at.n_ctx = d.n_ctx; at.ldS = a->ldS; at.B = B; at.pm = a->pm; at.pl = a->pl; at.ldP = a->ldP;
        if (single) {
            pa_launch_dep(pdl, pa_k_dec_scores, dim3(cdiv(n_kv_cap, PA_DS_KEYS)), dim3(256), pa_dec_scores_smem(H, G, dq), st, at, (const float *)a->qkv, (const float *)io.kc[li], io.pos_dev, a->S, io.err_dev, (int)cdiv(n_kv_cap, PA_DS_KEYS), (float *)nullptr);
            PA_LAUNCH();
            pa_launch_dep(pdl, pa_k_dec_pv, dim3(cdiv(dv, PA_DP_DIMS), G, pa_dec_pv_split(H, G)), dim3(256), pa_dec_pv_smem(H, G), st, at, (const float *)a->S, (const float *)io.vct[li], io.pos_dev, a->att, pa_dec_pv_chunk(H, G), io.err_dev);
            PA_LAUNCH();
        } else {
            pa_k_scores<<<dim3(cdiv(n_kv, PA_TN), cdiv(bs, PA_TM), H), blk, 0, st>>>(at, a->qkv, nqkv, io.kc[li], w.kd, a->S, io.pos_dev, bs, 0, (int)cdiv(n_kv, PA_TN));
            PA_LAUNCH();
            pa_k_mix_softmax<<<bs, 256, 4 * (size_t)H * H, st>>>(at, a->S, io.pos_dev, bs);
            PA_LAUNCH();
            pa_k_pv<<<dim3(cdiv(dv, PA_TN), cdiv(bs, PA_TM), H), blk, 0, st>>>(at, a->S, io.vct[li], a->att, w.od, io.pos_dev, bs);
            PA_LAUNCH();
        }
        if (single) {
            PaMv mv{};
            mv.x = a->att; mv.W = w.wo; mv.bias = w.bo; mv.N = dim; mv.K = w.od; mv.y = a->ao;
            if (!routed) mv.residual = a->x; // no feed-forward: the layer ends here
            mv.ksplit = pick_ksplit(dim, w.od); mv.prefetch = a->opt_prefetch;
            pa_launch_dep(pdl, pa_k_dec_mv<ROUND>, dim3(mv_grid(dim, mv.ksplit, w.od)), dim3(PA_DV_THREADS), 0, st, mv);
        } else if (tc) {
            int rc = tc_dense(a->att, w.od, bs, w.od, w.t_o, dim, w.bo, a->ao, dim);
            if (rc) return rc;
        } else {
            pa_k_linear<ROUND><<<dim3(cdiv(dim, PA_TN), cdiv(bs, PA_TM)), blk, 0, st>>>(a->att, w.od, w.wo, w.bo, a->ao, dim, bs, dim, w.od);
        }
        PA_LAUNCH();
        // ---- routed feed-forward on the same normed input
        int top = 0;
        if (routed) {
            top = l.top_k;
            const int ff = l.expert_ff;
            int rc = 0;
            if (!single) {
                pa_k_router<<<bs, 256, 0, st>>>(a->h, w.router, dim, pa_route_of(l), a->sel_e, a->sel_w, a->sgate);
                PA_LAUNCH();
            }
            if (single) {
                if (a->opt_fork) PA_CK(cudaStreamWaitEvent(st, a->ev_join, 0));
                const int ksd = pick_ksplit(dim, ff);
                pa_k_dec_expert_down<ROUND><<<cdiv(dim, PA_DV_ROWS / ksd), PA_DV_THREADS, 0, st>>>(a->y, a->sel_e, a->sel_w, top, w.wdown, a->ao, a->x, dim, ff, l.route_on_input, ksd);
                PA_LAUNCH();
            } else if ((rc = routed_batch(a->h, w))) {
                return rc;
            }
        }
        if (!single) {
            pa_k_combine<<<dim3(cdiv(dim, 256), bs), 256, 0, st>>>(a->x, a->ao, a->slot, top, dim);
            PA_LAUNCH();
        }
        if (a->taps_on) {
            if (!a->taps[(size_t)li]) { int rc = aalloc(a, (void **)&a->taps[(size_t)li], 4 * (size_t)dim * B, err); if (rc) return rc; }
            PA_CK(cudaMemcpyAsync(a->taps[(size_t)li], a->x, 4 * (size_t)dim * bs, cudaMemcpyDeviceToDevice, st));
        }
    }
    if (lm_head) {
        if (!single) {
            if (pend_y || groups > 1 || center) {
                int rc = seam(a->h, a->final_norm);
                if (rc) return rc;
            } else {
                pa_k_norm<<<bs, 256, 0, st>>>(a->h, a->x, a->final_norm, dim, d.norm_eps);
                PA_LAUNCH();
            }
        }
        if (single) {
            PaMv mv{};
            mv.x = a->x; mv.norm_w = a->final_norm; mv.eps = d.norm_eps; mv.W = a->head; mv.N = d.vocab_size; mv.K = dim; mv.y = a->logits;
            if (a->has_seq) seam_mv(mv, a->final_norm);
            mv.ksplit = pick_ksplit(d.vocab_size, dim); mv.prefetch = a->opt_prefetch;
            pa_launch_dep(pdl, pa_k_dec_mv<ROUND>, dim3(mv_grid(d.vocab_size, mv.ksplit, dim)), dim3(PA_DV_THREADS), 4 * (size_t)dim, st, mv);
        } else if (tc) {
            int rc = tc_dense(a->h, dim, bs, dim, a->t_head, d.vocab_size, nullptr, a->logits, d.vocab_size);
            if (rc) return rc;
        } else {
            pa_k_linear<ROUND><<<dim3(cdiv(d.vocab_size, PA_TN), cdiv(bs, PA_TM)), blk, 0, st>>>(a->h, dim, a->head, nullptr, a->logits, d.vocab_size, bs, d.vocab_size, dim);
        }
        PA_LAUNCH();
    }
    return 0;
}

int ps_arch_forward(PsArch *a, const PsArchIO &io, int bs, int pos0, int lm_head, std::string &err) {
    if (!a->bound) return afail(err, PS_CUDA_ERR_INVALID, "forward: no model bound");
    if (bs <= 0 || bs > a->d.max_batch || pos0 < 0 || pos0 + bs > a->d.n_ctx) return afail(err, PS_CUDA_ERR_INVALID, "forward: batch %d at position %d does not fit", bs, pos0);
    return a->round ? forward_t<true>(a, io, bs, pos0, lm_head, err) : forward_t<false>(a, io, bs, pos0, lm_head, err);
}
