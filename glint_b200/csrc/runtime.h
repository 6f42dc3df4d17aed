// The native step runtime: routed operations and the program executor.
//
// A model is lowered once into a program: a list of operations with fixed device pointers
// (weights, cache pages, the values between kernels) whose token counts and metadata pointers
// come from the step that runs it.  One call runs a whole step's worth of operations, choosing
// for each the kernel that its sizes ask for (the weight-streaming or the tiled product, the
// split or the tiled attention, the fused or the two-kernel q/k/v path).  The same routed
// operations are exported one by one, so that the Python path of a part and the program make the
// same choices by construction.  The reference's counterpart is the compiled forward pass and
// engine loop (src/transformer/forward.rs:450-522, src/server/engine.rs:449-671).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define GLINT_MAX_GROUPS 8

extern "C" {

// One step's shape and device metadata.  Device arrays are int32.
struct GlintStep {
  long long id;                 // increases with every step: what is computed once per step is marked with it
  int num_tokens, num_seqs, max_seq_len, max_context;
  int leading_single, leading_single_context, num_logit_rows, num_groups;
  int uneven;                   // how far the single tokens' contexts fall short of the longest: their sum is
                                // about (requests x longest) >> uneven
  const int* token_ids;         // [tokens]
  const int* positions;         // [tokens]
  const int* token_seq;         // [tokens] the token's request within the step = its block-table row
  const int* seq_slot;          // [requests]
  const int* seq_start;         // [requests] tokens cached before the step
  const int* cu_seqlens;        // [requests + 1]
  const int* logit_rows;        // [logit rows]
  const int* block_table[GLINT_MAX_GROUPS];   // per cache group: [requests][max_pages]
  int max_pages[GLINT_MAX_GROUPS];
};

// Entry points of the tensor-core library, bound at run time (a float32 process never loads it).
struct GlintTensorEntries {
  int (*gemm_tcgen05)(const void*, const void*, void*, int, int, int, int, long long, float, int, int, int, float*,
                      int*, int*, int, cudaStream_t);
  int (*gemm_skinny)(const void*, const void*, void*, int, int, int, int, float, int, int, int, cudaStream_t);
  int (*gemm_tcgen05_rope)(const void*, const void*, int, int, const float*, const int*, const int*, const int*, int,
                           void*, void*, void*, int, int, int, int, int, int, int*, cudaStream_t);
  int (*gemm_skinny_rope)(const void*, const void*, int, int, const int*, const int*, const int*, int, const float*,
                          float, void*, void*, void*, int, int, int, int, int, int*, cudaStream_t);
  int (*attention_decode)(const void*, const void*, const void*, const int*, const int*, const int*, int, void*, int,
                          int, int, int, int, int, float, float, int, int, int*, cudaStream_t);
  int (*attention_decode_stream_plan)(const int*, const int*, int, int, int, int, int, int, int, int, void*, int*,
                                      cudaStream_t);
  int (*attention_decode_stream)(const void*, const void*, const void*, const int*, const int*, const int*, int, void*,
                                 int, int, int, int, int, int, float, float, int, int, const void*, float*, int*, int,
                                 int*, cudaStream_t);
  int (*attention_prefill)(const void*, const void*, const void*, const int*, const int*, const int*, int, void*, int,
                           int, int, int, int, int, int, float, float, int, int*, cudaStream_t);
  int (*attention_tcgen05)(const void*, const void*, const void*, const int*, const int*, const int*, int, void*, int,
                           int, int, int, int, int, int, int, float, float, int, int*, cudaStream_t);
};

// Scratch of the single-token attention that shares the pages of a launch evenly among its blocks: the
// plans of a step (one for every window, page size and number of kv heads that its layers have; made by
// the first layer that asks and kept until the next step), the partial results and the arrival counters.
#define GLINT_ATTN_PLANS 8
struct GlintAttnScratch {
  int mode;                     // 0: the runtime chooses between the two single-token kernels; 1: this one wherever
                                // it takes the sizes; 2: never (tests and measurements)
  int early_off;                // 1: no page is started before the wait for the kernel in front (measurements)
  int blocks;                   // blocks of a launch (two per SM)
  void* starts;                 // [GLINT_ATTN_PLANS][blocks][2] int4
  int* headers;                 // [GLINT_ATTN_PLANS][2]
  float* partials;              // [partial_floats]
  long long partial_floats;
  int* arrive;                  // [arrive_ints], zero between launches
  int arrive_ints;
  int next;                     // the plan slot to fill next
  long long plan_step[GLINT_ATTN_PLANS];
  int plan_tokens[GLINT_ATTN_PLANS], plan_window[GLINT_ATTN_PLANS], plan_page[GLINT_ATTN_PLANS], plan_nkv[GLINT_ATTN_PLANS];
  int plan_hd[GLINT_ATTN_PLANS];
};

// What all operations of one model share.
struct GlintRuntime {
  int tensor_cores;             // bfloat16 with the tensor-core kernels (else the CUDA-core kernels)
  int dtype;                    // GLINT_DTYPE_* of activations, matrices and cache pages
  int sms;                      // streaming multiprocessors of the device
  int* status;                  // device status word
  float* workspace;             // split-K scratch of the tiled product
  int* counters;
  GlintAttnScratch* attn;       // null: single tokens always take the cluster kernel
  GlintTensorEntries tensor;
};

// A cache view as the attention operations see it.
struct GlintView {
  void* k;
  void* v;
  int page_size, num_pages, group, writes;
};

// The table of rotation angles of one rotary encoding: filled at most once per step.
struct GlintTrigTable {
  float* table;                 // [capacity tokens][rotary_dim / 2] (cos, sin)
  long long filled_step;
};

// ---- routed operations -------------------------------------------------------------------------------
// out [M, N] = a [M, K] w[N, K]^T (float32, or bfloat16 when gated); cap > 0: soft cap; gated: w is
// [2N, K] and out = act(a w[:N]^T) * (a w[N:]^T) in the activation dtype, `tmp` [M, 2N] float32 is used
// when no kernel fuses it.
int glint_op_linear(const GlintRuntime* rt, const void* a, const void* w, void* out, int out_bf16, int M, int N, int K,
                    float cap, int gated, int act, float* tmp, cudaStream_t stream);
// q, k, v = x w^T, rotary encoding of q and k, q to q_out, k and v into the pages of `view`.
int glint_op_qkv_rope(const GlintRuntime* rt, const GlintStep* step, const void* x, const void* w, void* q_out,
                      float* qkv_tmp, const GlintView* view, int nh, int nkv, int hd, int K, const float* inv_freq,
                      float factor, int rotary_dim, GlintTrigTable* trig, cudaStream_t stream);
// Rotary encoding of a finished q/k/v product and the cache write (the second half of the two-kernel path).
int glint_op_rope_store(const GlintRuntime* rt, const GlintStep* step, const float* qkv, void* q_out,
                        const GlintView* view, int nh, int nkv, int hd, const float* inv_freq, float factor,
                        int rotary_dim, cudaStream_t stream);
int glint_op_attention(const GlintRuntime* rt, const GlintStep* step, const void* q, const GlintView* view, void* out,
                       int nh, int nkv, int hd, float multiplier, float cap, int window, cudaStream_t stream);

// ---- which kernel a product takes (exported for tests and measurements) --------------------------------
// 0: CUDA-core product, 1: weight-streaming product, 2: tiled tensor-core product
int glint_route_linear(const GlintRuntime* rt, int M, int N, int K);

// Kernels launched so far through the routed operations and programs of this process.
long long glint_native_launches();
// Operations that a tensor-core runtime ran on CUDA cores because no tensor-core kernel takes their sizes.
long long glint_native_fallbacks();
int glint_decode_splits(int tokens, int nkv, int max_context, int uneven, int sms);
// 1 when single tokens of these counts take the kernel that shares all pages of the launch evenly among
// its blocks, 0 when every (token, kv head) gets a cluster of glint_decode_splits blocks.
int glint_decode_streams(int tokens, int nh, int nkv, int max_context, int uneven, int sms);

// ---- programs ------------------------------------------------------------------------------------------
struct GlintProgram;
enum GlintOpKind {
  GLINT_OP_EMBED = 1, GLINT_OP_RMSNORM = 2, GLINT_OP_ADD_RMSNORM = 3, GLINT_OP_LINEAR = 4, GLINT_OP_QKV_ROPE = 5,
  GLINT_OP_ROPE_STORE = 6, GLINT_OP_ATTENTION = 7, GLINT_OP_HOST = 8
};
// One operation: pointers in p, integers in i, floats in f; their meaning per kind is in runtime.cu.
struct GlintOp {
  int kind;
  int rows;                     // 0: one row per token of the step; 1: one row per wanted logit row
  void* p[10];
  long long i[10];
  float f[6];
};

GlintProgram* glint_program_create(const GlintRuntime* rt);
void glint_program_destroy(GlintProgram* prog);
int glint_program_add(GlintProgram* prog, const GlintOp* op);
int glint_program_size(const GlintProgram* prog);
// Runs operations [first, last) for `step`; returns 0 or an error code, with the failing operation in *failed.
int glint_program_run(GlintProgram* prog, const GlintStep* step, int first, int last, int* failed, cudaStream_t stream);

}  // extern "C"
