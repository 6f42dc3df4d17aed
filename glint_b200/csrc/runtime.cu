// Routed operations and the program executor (see runtime.h).  Host code only: every kernel is
// launched through the entry point of the file that holds it.
#include "runtime.h"

#include <vector>

#include "common.cuh"

extern "C" {
int glint_embed_scale(const void* table, int dtype, const int* ids, float* x, int T, int H, float scale, int vocab,
                      int* status, cudaStream_t stream);
int glint_rmsnorm(const float* x, const int* row_index, const float* w, void* out, int dtype, int rows, int H,
                  float eps, float offset, cudaStream_t stream);
int glint_add_rmsnorm(float* x, const float* y, const float* w_a, float eps_a, float offset_a, void* out, int dtype,
                      const float* w_b, float eps_b, float offset_b, int rows, int H, cudaStream_t stream);
int glint_rope_table(const int* positions, const float* inv_freq, float factor, float* out, int T, int half,
                     cudaStream_t stream);
int glint_rope_kv_write(const float* qkv, const int* positions, const int* token_slot, const int* block_table,
                        int max_pages, const float* inv_freq, float factor, int rot, void* q_out, void* k_pool,
                        void* v_pool, int dtype, int T, int nh, int nkv, int hd, int page_size, int num_pages,
                        int* status, cudaStream_t stream);
int glint_gated_act(const float* gu, void* out, int dtype, int T, int I, int act, cudaStream_t stream);
int glint_gemm_plain(const void* A, const void* W, int dtype, float* out, int M, int N, int K, float cap,
                     cudaStream_t stream);
int glint_attention_plain(const void* q, const void* k_pool, const void* v_pool, int dtype, const int* positions,
                          const int* token_slot, const int* block_table, int max_pages, void* out, int T, int nh,
                          int nkv, int hd, int page_size, int num_pages, float multiplier, float cap, int window,
                          int* status, cudaStream_t stream);
}

namespace {

long long g_launches = 0;     // kernels launched through the routed operations (one host thread drives a model)
long long g_fallbacks = 0;    // operations of a tensor-core runtime that took a CUDA-core kernel (sizes no other takes)
inline int counted(int rc) {
  ++g_launches;
  return rc;
}

// ---- which product kernel ------------------------------------------------------------------------------
constexpr int SKINNY_MAX_TOKENS = 16;
constexpr long long SKINNY_MAX_FEATURES = 65536;     // beyond this the tiled kernel streams at the memory's speed anyway
constexpr long long SKINNY_WIDE_LIMIT = 12ll << 20;  // 9 to 16 tokens: only products whose launch cost outweighs their stream

bool tiled_supported(int M, int N, int K) { return M > 0 && N > 0 && K > 0 && K % 8 == 0; }
bool skinny_supported(int M, int N, int K) { return M >= 1 && M <= 16 && N >= 1 && K >= 64 && K % 64 == 0; }
// Few tokens go to the weight-streaming kernel: up to 8 always, 9 to 16 when the matrix is small.
// The widest matrices stream as fast or faster through the tiled kernel whatever the tokens (measured in a
// decode step of 8 requests: 51 M weights, the 9B shape's feed-forward, 1.29 -> 1.25 ms for 8 layers; 170 M, the
// 27B shape's, 1.51 -> 1.48 ms for 4; no difference at one request)
constexpr long long SKINNY_MAX_WEIGHTS = 45ll << 20;
bool takes_skinny(int M, long long N, int K) {
  if (M > SKINNY_MAX_TOKENS || N > SKINNY_MAX_FEATURES || !skinny_supported(M, (int)N, K)) return false;
  if (N * K > SKINNY_MAX_WEIGHTS) return false;
  return M <= 8 || N * K <= SKINNY_WIDE_LIMIT;
}

// ---- which attention kernel -----------------------------------------------------------------------------
// as glint_attention_decode_supported (the tensor-core library is not linked here): three stages of a page of
// keys and values have to fit a block's shared memory
bool decode_supported(int nh, int nkv, int hd, int page) {
  if (!(nkv > 0 && nh % nkv == 0 && hd % 16 == 0 && hd >= 16 && hd <= 256 && page % 16 == 0 && page >= 16 && page <= 256))
    return false;
  const long long page_bytes = (long long)((hd + 63) / 64) * page * 128;
  const int G = nh / nkv, HP = G < 8 ? G : 8;
  return 3 * 2 * page_bytes + 3ll * HP * (hd + 2) * 4 + (long long)G * (hd + 2) * 4 + 2048 <= 227 * 1024;
}
bool prefill_supported(int nh, int nkv, int hd) {
  return nkv > 0 && nh % nkv == 0 && nh / nkv <= 64 && hd % 16 == 0 && hd >= 16 && hd <= 256;
}
bool tiled_attention_supported(int nh, int nkv, int hd, int page) {
  return nkv > 0 && nh % nkv == 0 && nh / nkv <= 128 && hd % 16 == 0 && hd >= 16 && hd <= 256 &&
         (page == 16 || page == 32 || page == 64);
}
constexpr int SPLIT_SINGLES_FROM = 4096;   // context from which single tokens in front of portions leave the tiled kernel
constexpr int SPLIT_SINGLES_UP_TO = 8;     // so few of them leave it at any context

}  // namespace

// Blocks for about one wave (2 fit on each SM), each split with at least 128 keys; the splits of a token
// are one thread-block cluster: a power of two up to 8 (measured: clusters of 9 to 16 blocks, or of 6,
// take 1.5 times as long when there are many of them), 16 only for one or two requests, where nothing
// else puts more SMs to work.
extern "C" int glint_decode_splits(int tokens, int nkv, int max_context, int uneven, int sms) {
  const int rows = tokens * nkv > 1 ? tokens * nkv : 1;
  const int want = 2 * sms / rows;
  const int limit = tokens * nkv <= 8 ? 16 : 8;
  const int most = max_context / 128 < limit ? max_context / 128 : limit;
  int splits = want < most ? want : most;
  if (splits < 1) splits = 1;
  while (splits & (splits - 1)) splits &= splits - 1;
  // All clusters of the launch should be on the SMs at once: a cluster stays within one of the 8 GPCs, two
  // blocks fit an SM, and not every GPC has its full share of the SMs (counted here as two fewer), so 148
  // SMs hold 32 clusters of 8 but not the 36 of 9 requests with 4 kv heads (35 us with 8 splits against 29 us
  // with 4), and 64 clusters of 4 but not the 72 of 9 requests with 8 kv heads (58 us against 34 us for 64).
  while (splits > 1 && tokens * nkv > 8 * ((2 * (sms / 8 - 2)) / splits)) splits >>= 1;
  if (uneven > 0) {
    // Contexts of different lengths: a block streams about 32 GB/s whatever else runs (its ring of pages
    // against the memory's latency), so the launch lasts as long as its longest block, and the blocks of
    // the short contexts leave their SMs early.  More splits shorten the longest block: as many as keep it
    // under the time the whole launch needs at full bandwidth, which is what the rule above gives for
    // (rows >> uneven) rows of the longest context.  56 requests of 200 to 4600 keys, 4 kv heads: 176 us
    // with one split, 138 us with 4; 24 requests with 8 kv heads: 174 and 106 us.
    const int eff = (rows >> uneven) > 1 ? (rows >> uneven) : 1;
    int more = 1;
    while (more < most && more * eff * 10 < 21 * sms) more <<= 1;      // more >= 2.1 sms / eff, a power of two
    while (more > most) more >>= 1;
    if (more > splits) splits = more;
  }
  return splits;
}

// Which kernel single tokens take.  A cluster per (token, kv head) is the faster way while the contexts are
// even and the clusters fill the SMs (8 requests x 4 kv heads x 8 splits, whole decode steps of the 2B shape:
// 1.806 against 1.833 ms; 16 x 4 x 4: 2.304 against 2.347; one request: 1.512 against 1.547).  The kernel that
// shares all pages of the launch evenly wins where the clusters' power of two leaves SMs idle (12 requests:
// 2.175 against 2.235 ms; 24: 2.81 against 3.02; 48: 3.78 against 4.155), where single blocks make more than
// one wave (64 requests x 8 kv heads, 9B shape: 12.19 against 12.39 ms), and where contexts are uneven, since a
// block per pair waits for the longest (serving 64 requests of 128 to 4,600 tokens, 9B shape: decode steps
// of 57 to 64 requests 11.8 against 13.6 ms, of 9 to 16 requests 6.0 against 7.1 ms).
extern "C" int glint_decode_streams(int tokens, int nh, int nkv, int max_context, int uneven, int sms) {
  if (nkv <= 0 || nh / nkv > 8 || tokens > 1024) return 0;
  const int pairs = tokens * nkv;
  if (pairs > 2 * sms) return 1;
  if (uneven > 0) return pairs >= 32 ? 1 : 0;
  return pairs >= 16 && pairs * glint_decode_splits(tokens, nkv, max_context, 0, sms) * 10 <= 7 * 2 * sms ? 1 : 0;
}

extern "C" int glint_route_linear(const GlintRuntime* rt, int M, int N, int K) {
  if (!rt->tensor_cores || rt->dtype != GLINT_DTYPE_BF16 || !tiled_supported(M, N, K)) return 0;
  return takes_skinny(M, N, K) ? 1 : 2;
}

extern "C" int glint_op_linear(const GlintRuntime* rt, const void* a, const void* w, void* out, int out_bf16, int M,
                               int N, int K, float cap, int gated, int act, float* tmp, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return GLINT_OK;
  const int route = glint_route_linear(rt, M, N, K);
  if (route == 1)
    return counted(rt->tensor.gemm_skinny(a, w, out, gated ? 1 : out_bf16, M, N, K, gated ? 0.f : cap, gated, gated ? N : 0,
                                  act, stream));
  if (route == 2)
    return counted(rt->tensor.gemm_tcgen05(a, w, out, gated ? 1 : out_bf16, M, N, K, gated ? 2ll * N : (long long)N,
                                   gated ? 0.f : cap, gated, gated ? N : 0, act, rt->workspace, rt->counters,
                                   rt->status, 0, stream));
  // CUDA cores: float32 results; a gated product goes through `tmp` [M, 2N]
  if (rt->tensor_cores) ++g_fallbacks;
  if (out_bf16 && !gated) return GLINT_ERR_BAD_ARG;
  if (!gated) return counted(glint_gemm_plain(a, w, rt->dtype, (float*)out, M, N, K, cap, stream));
  if (!tmp) return GLINT_ERR_BAD_ARG;
  const int rc = counted(glint_gemm_plain(a, w, rt->dtype, tmp, M, 2 * N, K, 0.f, stream));
  if (rc != GLINT_OK) return rc;
  return counted(glint_gated_act(tmp, out, rt->dtype, M, N, act, stream));
}

extern "C" int glint_op_rope_store(const GlintRuntime* rt, const GlintStep* step, const float* qkv, void* q_out,
                                   const GlintView* view, int nh, int nkv, int hd, const float* inv_freq,
                                   float factor, int rotary_dim, cudaStream_t stream) {
  return counted(glint_rope_kv_write(qkv, step->positions, step->token_seq, step->block_table[view->group],
                             step->max_pages[view->group], inv_freq, factor, rotary_dim, q_out,
                             view->writes ? view->k : nullptr, view->writes ? view->v : nullptr, rt->dtype,
                             step->num_tokens, nh, nkv, hd, view->page_size, view->num_pages, rt->status, stream));
}

extern "C" int glint_op_qkv_rope(const GlintRuntime* rt, const GlintStep* step, const void* x, const void* w,
                                 void* q_out, float* qkv_tmp, const GlintView* view, int nh, int nkv, int hd, int K,
                                 const float* inv_freq, float factor, int rotary_dim, GlintTrigTable* trig,
                                 cudaStream_t stream) {
  const int M = step->num_tokens;
  if (M <= 0) return GLINT_OK;
  const int g = view->group;
  void* k = view->writes ? view->k : nullptr;
  void* v = view->writes ? view->v : nullptr;
  if (rt->tensor_cores && rt->dtype == GLINT_DTYPE_BF16) {
    // one kernel for a few single tokens: the weight-streaming product with the rotation in its epilogue
    if (M <= SKINNY_MAX_TOKENS && K >= 64 && K % 64 == 0 && hd % 16 == 0 && hd >= 16 && rotary_dim == hd)
      return counted(rt->tensor.gemm_skinny_rope(x, w, M, K, step->positions, step->token_seq, step->block_table[g],
                                         step->max_pages[g], inv_freq, factor, q_out, k, v, nh, nkv, hd,
                                         view->page_size, view->num_pages, rt->status, stream));
    // one kernel for portions: the tiled product with the rotation in its epilogue.  Its grid is heads x
    // token tiles with K unsplit, so it wants tiles for half of the SMs; head sizes in steps of 256.
    const int heads = view->writes ? nh + 2 * nkv : nh;
    const int min_blocks = rt->sms / 2;
    if (trig && K % 8 == 0 && hd >= 256 && hd % 256 == 0 && rotary_dim == hd &&
        (long long)heads * (hd / 256) * ((M + 127) / 128) >= min_blocks) {
      if (trig->filled_step != step->id) {       // the angles of this step's tokens, once for all layers
        const int rc = counted(glint_rope_table(step->positions, inv_freq, factor, trig->table, M, rotary_dim / 2, stream));
        if (rc != GLINT_OK) return rc;
        trig->filled_step = step->id;
      }
      return counted(rt->tensor.gemm_tcgen05_rope(x, w, M, K, trig->table, step->positions, step->token_seq,
                                          step->block_table[g], step->max_pages[g], q_out, k, v, nh, nkv, hd,
                                          view->page_size, view->num_pages, min_blocks, rt->status, stream));
    }
  }
  if (!qkv_tmp) return GLINT_ERR_BAD_ARG;
  const int rc = glint_op_linear(rt, x, w, qkv_tmp, 0, M, (nh + 2 * nkv) * hd, K, 0.f, 0, 0, nullptr, stream);
  if (rc != GLINT_OK) return rc;
  return glint_op_rope_store(rt, step, qkv_tmp, q_out, view, nh, nkv, hd, inv_freq, factor, rotary_dim, stream);
}

// Attention of the first `T` tokens of the step, single tokens all: the stream kernel with this step's plan
// for (window, page size, kv heads), made here if no earlier layer of the step has, or the cluster kernel.
static int decode_attention(const GlintRuntime* rt, const GlintStep* step, const void* q, const GlintView* view,
                            void* out, int T, int nh, int nkv, int hd, float multiplier, float cap, int window,
                            cudaStream_t stream) {
  const GlintTensorEntries& t = rt->tensor;
  const int g = view->group;
  const int* table = step->block_table[g];
  const int max_pages = step->max_pages[g];
  const int page = view->page_size;
  GlintAttnScratch* a = rt->attn;
  const bool wanted = a && (a->mode == 1 ? (nkv > 0 && nh / nkv <= 8 && T <= 1024)
                                         : a->mode == 0 && glint_decode_streams(T, nh, nkv, step->max_context,
                                                                                 step->uneven, rt->sms));
  if (wanted && t.attention_decode_stream &&
      (long long)a->blocks * 2 * (nh / nkv) * (hd + 4) <= a->partial_floats && (long long)T * nkv <= a->arrive_ints) {
    int slot = -1;
    for (int i = 0; i < GLINT_ATTN_PLANS; ++i)
      if (a->plan_step[i] == step->id && a->plan_tokens[i] == T && a->plan_window[i] == window &&
          a->plan_page[i] == page && a->plan_nkv[i] == nkv && a->plan_hd[i] == hd)
        slot = i;
    void* starts = nullptr;
    // A plan that an earlier layer of the step made lies several kernels back: the producer warps may read it
    // and start their first pages before they wait for the kernel in front (which writes only the tokens'
    // newest keys and values: the tokens here are single tokens of different requests).
    const int early = slot >= 0 ? 1 : 0;
    if (slot < 0) {
      slot = a->next;
      a->next = (a->next + 1) % GLINT_ATTN_PLANS;
      starts = (char*)a->starts + (size_t)slot * a->blocks * 32;
      const int rc = counted(t.attention_decode_stream_plan(step->positions, step->token_seq, T, window, page, hd, nkv,
                                                            a->blocks, 8, -1, starts, a->headers + 2 * slot, stream));
      if (rc != GLINT_OK) return rc;
      a->plan_step[slot] = step->id;
      a->plan_tokens[slot] = T;
      a->plan_window[slot] = window;
      a->plan_page[slot] = page;
      a->plan_nkv[slot] = nkv;
      a->plan_hd[slot] = hd;
    }
    starts = (char*)a->starts + (size_t)slot * a->blocks * 32;
    return counted(t.attention_decode_stream(q, view->k, view->v, step->positions, step->token_seq, table, max_pages, out,
                                             T, nh, nkv, hd, page, view->num_pages, multiplier, cap, window, a->blocks,
                                             starts, a->partials, a->arrive, a->early_off ? 0 : early, rt->status,
                                             stream));
  }
  return counted(t.attention_decode(q, view->k, view->v, step->positions, step->token_seq, table, max_pages, out, T, nh,
                                    nkv, hd, page, view->num_pages, multiplier, cap, window,
                                    glint_decode_splits(T, nkv, step->max_context, step->uneven, rt->sms), rt->status,
                                    stream));
}

extern "C" int glint_op_attention(const GlintRuntime* rt, const GlintStep* step, const void* q, const GlintView* view,
                                  void* out, int nh, int nkv, int hd, float multiplier, float cap, int window,
                                  cudaStream_t stream) {
  const int T = step->num_tokens;
  if (T <= 0) return GLINT_OK;
  const int g = view->group;
  const int* table = step->block_table[g];
  const int max_pages = step->max_pages[g];
  const int page = view->page_size;
  const bool dec = decode_supported(nh, nkv, hd, page), pre = prefill_supported(nh, nkv, hd);
  if (rt->tensor_cores && !(dec || pre)) ++g_fallbacks;
  if (!(rt->tensor_cores && rt->dtype == GLINT_DTYPE_BF16 && (dec || pre)))
    return counted(glint_attention_plain(q, view->k, view->v, rt->dtype, step->positions, step->token_seq, table, max_pages,
                                 out, T, nh, nkv, hd, page, view->num_pages, multiplier, cap, window, rt->status,
                                 stream));
  const GlintTensorEntries& t = rt->tensor;
  if (step->max_seq_len > 1 && tiled_attention_supported(nh, nkv, hd, page)) {
    const int lead = step->leading_single;
    // What the single tokens in front would cost in the tiled kernel.  Walks: a block of 128 rows for each token
    // and kv head, two to eight rows of it in use, takes about 3 us of an SM per tile of 128 keys.  Slots: the
    // grid has a block for every (query tile of the longest portion, request, kv head), and a block that finds
    // its request shorter than that leaves after one load, about 1.8 us of an SM each.
    const int G = nh / nkv;
    const long long walks = (((long long)lead * ((step->leading_single_context + 127) / 128)) >> step->uneven) * nkv;
    const long long slots = (long long)lead * ((step->max_seq_len * G + 127) / 128) * nkv;
    if (lead > 0 && dec && (lead <= SPLIT_SINGLES_UP_TO || step->leading_single_context >= SPLIT_SINGLES_FROM ||
                            walks >= 4ll * rt->sms || slots >= 8ll * rt->sms)) {
      // Decoding requests in front of the prompt portions: in the tiled kernel one block walks all keys of
      // such a row (8192 keys: 150 us, and the step waits for it), and many rows take the SMs from the
      // portions' tiles (48 requests of 2400 keys beside a portion of 4048 tokens, 8 kv heads: 494 us, of which
      // the portion needs 176; 16 requests beside 4080 tokens: 290 us, of which 100 go to blocks that only find
      // out that they have nothing to do); the single-token kernels stream them at the memory's speed instead.
      // A few requests with short contexts beside short portions stay: their walks hide behind the portions' tiles.
      // The portions keep their absolute token offsets.
      int rc = decode_attention(rt, step, q, view, out, lead, nh, nkv, hd, multiplier, cap, window, stream);
      if (rc != GLINT_OK) return rc;
      return counted(t.attention_tcgen05(q, view->k, view->v, step->cu_seqlens + lead, step->seq_start + lead,
                                 table + (size_t)lead * max_pages, max_pages, out, T, step->num_seqs - lead,
                                 step->max_seq_len, nh, nkv, hd, page, view->num_pages, multiplier, cap, window,
                                 rt->status, stream));
    }
    return counted(t.attention_tcgen05(q, view->k, view->v, step->cu_seqlens, step->seq_start, table, max_pages, out, T,
                               step->num_seqs, step->max_seq_len, nh, nkv, hd, page, view->num_pages, multiplier, cap,
                               window, rt->status, stream));
  }
  if ((step->max_seq_len > 1 || !dec) && pre)
    return counted(t.attention_prefill(q, view->k, view->v, step->cu_seqlens, step->seq_start, table, max_pages, out,
                               step->num_seqs, step->max_seq_len, nh, nkv, hd, page, view->num_pages, multiplier, cap,
                               window, rt->status, stream));
  return decode_attention(rt, step, q, view, out, T, nh, nkv, hd, multiplier, cap, window, stream);
}

// ---- programs ---------------------------------------------------------------------------------------------
struct GlintProgram {
  const GlintRuntime* rt;
  std::vector<GlintOp> ops;
};

extern "C" GlintProgram* glint_program_create(const GlintRuntime* rt) {
  GlintProgram* p = new GlintProgram();
  p->rt = rt;
  return p;
}

extern "C" void glint_program_destroy(GlintProgram* prog) { delete prog; }

extern "C" int glint_program_add(GlintProgram* prog, const GlintOp* op) {
  if (!prog || !op || op->kind < GLINT_OP_EMBED || op->kind > GLINT_OP_HOST) return GLINT_ERR_BAD_ARG;
  prog->ops.push_back(*op);
  return (int)prog->ops.size() - 1;
}

// Kernels launched so far through the routed operations and programs of this process.
extern "C" long long glint_native_launches() { return g_launches; }
// Operations that a runtime with tensor-core kernels ran on CUDA cores because of their sizes (K not a
// multiple of 8, a head size above 256 or not a multiple of 16): right, but far slower.
extern "C" long long glint_native_fallbacks() { return g_fallbacks; }

extern "C" int glint_program_size(const GlintProgram* prog) { return prog ? (int)prog->ops.size() : 0; }

// Per kind, what the fields of an operation hold:
//   EMBED        p: table, out            i: table dtype, H, vocab                    f: scale
//   RMSNORM      p: x, weight, out        i: out dtype, H                             f: eps, offset
//   ADD_RMSNORM  p: x, y, w_a, out, w_b   i: out dtype, H                             f: eps_a, offset_a, eps_b, offset_b
//   LINEAR       p: a, w, out, tmp        i: out bf16, N, K, gated, activation        f: cap
//   QKV_ROPE     p: x, w, q_out, tmp, view, inv_freq, trig   i: nh, nkv, hd, K, rotary dim    f: factor
//   ROPE_STORE   p: qkv, q_out, view, inv_freq               i: nh, nkv, hd, rotary dim       f: factor
//   ATTENTION    p: q, view, out          i: nh, nkv, hd, window                      f: multiplier, cap
//   HOST         nothing: the place of a step that the host language runs between two native stretches
// rows = 1: the operation runs on the wanted logit rows (RMSNORM gathers them from x, LINEAR takes that many).
extern "C" int glint_program_run(GlintProgram* prog, const GlintStep* step, int first, int last, int* failed,
                                 cudaStream_t stream) {
  if (!prog || !step || first < 0 || last > (int)prog->ops.size()) return GLINT_ERR_BAD_ARG;
  const GlintRuntime* rt = prog->rt;
  const int T = step->num_tokens;
  for (int n = first; n < last; ++n) {
    const GlintOp& op = prog->ops[n];
    const int rows = op.rows ? step->num_logit_rows : T;
    int rc = GLINT_OK;
    switch (op.kind) {
      case GLINT_OP_EMBED:
        rc = counted(glint_embed_scale(op.p[0], (int)op.i[0], step->token_ids, (float*)op.p[1], T, (int)op.i[1], op.f[0],
                               (int)op.i[2], rt->status, stream));
        break;
      case GLINT_OP_RMSNORM:
        rc = counted(glint_rmsnorm((const float*)op.p[0], op.rows ? step->logit_rows : nullptr, (const float*)op.p[1], op.p[2],
                           (int)op.i[0], rows, (int)op.i[1], op.f[0], op.f[1], stream));
        break;
      case GLINT_OP_ADD_RMSNORM:
        rc = counted(glint_add_rmsnorm((float*)op.p[0], (const float*)op.p[1], (const float*)op.p[2], op.f[0], op.f[1], op.p[3],
                               (int)op.i[0], (const float*)op.p[4], op.f[2], op.f[3], rows, (int)op.i[1], stream));
        break;
      case GLINT_OP_LINEAR:
        rc = glint_op_linear(rt, op.p[0], op.p[1], op.p[2], (int)op.i[0], rows, (int)op.i[1], (int)op.i[2], op.f[0],
                             (int)op.i[3], (int)op.i[4], (float*)op.p[3], stream);
        break;
      case GLINT_OP_QKV_ROPE:
        rc = glint_op_qkv_rope(rt, step, op.p[0], op.p[1], op.p[2], (float*)op.p[3], (const GlintView*)op.p[4],
                               (int)op.i[0], (int)op.i[1], (int)op.i[2], (int)op.i[3], (const float*)op.p[5], op.f[0],
                               (int)op.i[4], (GlintTrigTable*)op.p[6], stream);
        break;
      case GLINT_OP_ROPE_STORE:
        rc = glint_op_rope_store(rt, step, (const float*)op.p[0], op.p[1], (const GlintView*)op.p[2], (int)op.i[0],
                                 (int)op.i[1], (int)op.i[2], (const float*)op.p[3], op.f[0], (int)op.i[3], stream);
        break;
      case GLINT_OP_ATTENTION:
        rc = glint_op_attention(rt, step, op.p[0], (const GlintView*)op.p[1], op.p[2], (int)op.i[0], (int)op.i[1],
                                (int)op.i[2], op.f[0], op.f[1], (int)op.i[3], stream);
        break;
      case GLINT_OP_HOST:
        break;
      default:
        rc = GLINT_ERR_BAD_ARG;
    }
    if (rc != GLINT_OK) {
      if (failed) *failed = n;
      return rc;
    }
  }
  return GLINT_OK;
}
