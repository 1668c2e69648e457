// ps_arch.h - internal interface between the context (ps_cuda.cu: stream, cache sets / sessions, forward front end, sampling)
// and the layer-list model executor (ps_arch.cu: weights, workspace and kernels of models described layer by layer).
#pragma once
#include "../../include/ps_cuda.h"

#include <cuda_runtime.h>

#include <string>

struct PsArch; // weights + workspace + per-layer tables of one bound layer-list model

// what a forward pass gets from the context: the stream, the staged tokens / positions, the ACTIVE cache set
struct PsArchIO {
    cudaStream_t stream;
    const int32_t *tokens_dev; // [bs]
    const int32_t *pos_dev;    // [bs], consecutive
    float *const *kc;          // per layer: K rows  [n_ctx][n_kv_heads * qk_dim]
    float *const *vct;         // per layer: V^T rows [n_kv_heads * v_dim][n_ctx]
    int64_t *n_launch;         // the context's kernel-launch counter
    int *err_dev;              // the context's device-side failure flags ([0]: a tensor-core pipeline wait gave up)
    int n_kv_cap;              // > 0: size the single-token attention grid for this many keys (a captured step is replayed at any position)
};

int ps_arch_create(PsArch **out, const ps_cuda_arch_desc *desc, std::string &err);
void ps_arch_destroy(PsArch *a);
// bytes of one layer's K rows / V^T rows in a cache set (the context allocates them, per session)
size_t ps_arch_k_bytes(const PsArch *a, int layer);
size_t ps_arch_v_bytes(const PsArch *a, int layer);
int ps_arch_bind(PsArch *a, const ps_cuda_arch_weights *w, cudaStream_t stream, std::string &err);
// one forward pass over bs consecutive positions starting at pos0 (host copy of pos_dev[0]); logits [bs][vocab] fp32 land
// in ps_arch_logits() when lm_head != 0
int ps_arch_forward(PsArch *a, const PsArchIO &io, int bs, int pos0, int lm_head, std::string &err);
float *ps_arch_logits(PsArch *a);
void ps_arch_set_taps(PsArch *a, int on);
const float *ps_arch_tap(PsArch *a, int layer); // [max_batch][dim] of the last forward, nullptr when taps are off
int ps_arch_set_option(PsArch *a, const char *name, int value); // 1 = known option
// the single-token step reads the position from device memory only (it may be captured once and replayed)
bool ps_arch_step_replayable(const PsArch *a);
// some layer carries state that cannot be cut back to an earlier position (recurrences, convolution tails)
bool ps_arch_has_state(const PsArch *a);
