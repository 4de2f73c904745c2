// Task-graph compiler (host).  See task_graph.h.
#include "task_graph.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <set>
#include <sstream>

namespace mpk {
namespace {

constexpr int kSmemBudget = 232448;   // 227 KB opt-in dynamic shared memory per CTA on sm_100
constexpr int kMiscBytesHost = 1536;   // barriers, descriptors, flags (1 KB) + the attention stash ring
constexpr int ST_META = 0;            // batch description written by the batching task
constexpr int ST_META_OUT = 1;        // output_tokens (written by argmax, read by the batching task)

int elt_size(int dtype) {
  switch (dtype) {
    case MPK_BF16: case MPK_F16: case MPK_I16: return 2;
    case MPK_F32: case MPK_I32: case MPK_U32: return 4;
    case MPK_I64: case MPK_U64: return 8;
    default: return 1;
  }
}

int float_bits(float f) {
  int i;
  std::memcpy(&i, &f, 4);
  return i;
}


struct Builder {
  GraphInputs in;
  CompiledGraph *g;
  int64_t exchange_base_words = 0;   // start of the argmax-exchange area inside an inbox buffer
  std::string *err;
  const mpk_config &cfg;
  const std::vector<TensorInfo> &T;
  std::vector<LayerInfo> &L;
  int W;
  int nb_max;
  std::vector<std::vector<TaskDesc>> per_worker;
  std::vector<std::vector<int>> per_worker_exec;
  int rot = 0;

  Builder(GraphInputs i, CompiledGraph *out, std::string *e)
      : in(i), g(out), err(e), cfg(*i.cfg), T(*i.tensors), L(*i.layers), W(i.num_workers) {
    nb_max = std::min(std::max(cfg.max_num_batched_tokens, 1), (int)kMaxLinearTokens);
  }

  // largest activation tile: 64 KB up to 8 tokens (three 64 KB weight stages remain), 129 KB beyond (two 32 KB stages)
  int64_t x_tile_cap() const { return nb_max <= 8 ? 64 * 1024 + 256 : 64 * (1024 * 2 + kRowPadBytes); }

  // Does the graph run on the general instantiation of the megakernel (more than 8 batched tokens, or any FP8 /
  // expert / latent-attention / sampling layer)?
  bool general_graph() const {
    if (nb_max > 8 || cfg.max_num_batched_tokens > 8) return true;
    for (const auto &l : L)
      if (l.op >= MPK_OP_QUANTIZE_FP8) return true;
    return false;
  }

  // More than 8 batched tokens: bf16 linears whose K is a multiple of 64 run on tcgen05 (swap-AB, weights = M = 128,
  // tokens = N = tc_np() <= 64).  The activation operand tile is [K / 64][tc_np()][128 bytes], swizzled.
  // Graphs without a batching task: test mode, and online_notoken (one forward per call on a batch description the
  // caller manages; include/mirage/persistent_kernel/persistent_kernel.cuh:370-411 is the reference's counterpart).
  bool no_batch_task() const { return cfg.test_mode || cfg.mode == MPK_MODE_ONLINE_NOTOKEN; }
  int tc_np() const { return (nb_max + 15) / 16 * 16; }
  bool tc_linear(int64_t K) const { return nb_max > 8 && K % kTcKBlock == 0; }
  // FP8 linears on tcgen05 (block-scaled MMA): K a multiple of 512 (one packed scale word spans 512 columns).  The
  // operand tile is [KT / 128][tc_np()][128 bytes]; behind it sit the scale words of the k tile: 512 bytes per 512
  // columns for the activations and for each of up to kTcFp8MaxTiles row tiles.
  bool tc_linear_fp8(int64_t K) const { return nb_max > 8 && K % 512 == 0; }
  int64_t fp8_tc_tile_bytes(int64_t KT) const { return (int64_t)tc_np() * KT + (int64_t)(kTcFp8MaxTiles + 1) * KT; }
  // The e4m3 activation tile with its scale words may run on into the partial-sum area that follows the tile buffer
  // (these tasks keep no partial sums there), and the buffer may grow until five 16 KB ring slots remain (what the
  // 129 KB bf16 tile leaves as well): at 64 tokens that admits k tiles of 2048 instead of 1024, i.e. half as many
  // stage / drain pauses per task.
  static int64_t fp8_tc_tile_cap() { return (kSmemBudget - kMiscBytesHost - kPartialBytes - 5 * kTcSlotBytes) / 256 * 256; }
  int64_t linear_tile_bytes(int64_t K) const {
    return tc_linear(K) ? (int64_t)tc_np() * K * 2 : (int64_t)nb_max * (K * 2 + kRowPadBytes);
  }

  // activation tile of an FP8 linear: [tokens, KT] e4m3 rows padded by 16 bytes, then one scale exponent per
  // (token, 128-group) and per (weight row of the task, 128-group)
  static int64_t fp8_tile_bytes(int ntok, int64_t KT) {
    return (int64_t)ntok * (KT + kRowPadBytes) + 16 + (int64_t)ntok * (KT / 128) + 16 + (int64_t)kFp8TaskRows * (KT / 128) + 16;
  }

  // activation tile of an FP8 expert projection: as above, with the float32 scales kept raw (4 bytes each)
  static int64_t moe_fp8_tile_bytes(int ntok, int64_t KT) {
    return (int64_t)ntok * (KT + kRowPadBytes) + 16 + 4 * ((int64_t)ntok * (KT / 128) + 4) + 4 * (int64_t)kFp8TaskRows * (KT / 128) + 16;
  }

  int fail(int code, const std::string &msg) {
    *err = msg;
    return code;
  }

  // inputs / outputs (tensor ids) of a layer, after folding
  void layer_io(const LayerInfo &l, std::vector<int> *ins, std::vector<int> *outs) const {
    auto add = [](std::vector<int> *v, int t) { if (t >= 0) v->push_back(t); };
    switch (l.op) {
      case MPK_OP_EMBED: add(ins, l.t[0]); add(ins, l.t[1]); add(outs, l.t[2]); break;
      case MPK_OP_RMSNORM: add(ins, l.t[0]); add(ins, l.t[1]); add(outs, l.t[2]); break;
      case MPK_OP_RMSNORM_LINEAR:
        add(ins, l.t[0]); add(ins, l.t[1]); add(ins, l.t[2]); add(outs, l.t[3]); break;
      case MPK_OP_LINEAR: case MPK_OP_SPLITK_LINEAR: case MPK_OP_LINEAR_RESIDUAL: {
        if (l.gather_ar >= 0) {   // the activations arrive through the inbox; the layer materialises them
          add(ins, l.gather_res);
          add(outs, l.gather_out);
        } else {
          add(ins, l.prologue == PRO_PLAIN ? l.t[0] : l.pro_src);
        }
        if (l.prologue == PRO_RMSNORM) add(ins, l.pro_gamma);
        add(ins, l.t[1]);
        const int y = l.op == MPK_OP_LINEAR_RESIDUAL ? l.t[3] : l.t[2];
        if (l.op == MPK_OP_LINEAR_RESIDUAL) add(ins, l.t[2]);
        if (l.op == MPK_OP_SPLITK_LINEAR) add(ins, y);
        if (!l.push) add(outs, l.silu_out >= 0 ? l.silu_out : y);
        break;
      }
      case MPK_OP_ATTENTION: case MPK_OP_PAGED_ATTENTION:
        for (int i = 0; i < 7; ++i) add(ins, l.t[i]);
        add(outs, l.t[1]); add(outs, l.t[2]); add(outs, l.t[7]);
        break;
      case MPK_OP_SILU_MUL: add(ins, l.t[0]); add(outs, l.t[1]); break;
      case MPK_OP_AR_PUSH: add(ins, l.t[0]); break;
      case MPK_OP_ALLREDUCE: {
        if (l.ar_producer < 0) {   // before plan_allreduce(): plain reader of its input
          add(ins, l.t[0]);
        } else {                   // fused: reads the producer's residual, the partials arrive by push
          const LayerInfo &p = L[l.ar_producer];
          if (p.op == MPK_OP_LINEAR_RESIDUAL) add(ins, p.t[2]);
          if (p.op == MPK_OP_SPLITK_LINEAR) add(ins, p.t[2]);
        }
        add(outs, l.t[2]);
        break;
      }
      case MPK_OP_ARGMAX_PARTIAL: case MPK_OP_SAMPLING_PARTIAL:
        add(ins, l.t[0]); add(outs, l.t[1]); add(outs, l.t[2]); break;
      case MPK_OP_ARGMAX_REDUCE: case MPK_OP_SAMPLING_REDUCE: case MPK_OP_ARGMAX_EXCHANGE:
        add(ins, l.t[0]); add(ins, l.t[1]); add(outs, l.t[2]); break;
      case MPK_OP_ELEMENTWISE_ADD: add(ins, l.t[0]); add(ins, l.t[1]); add(outs, l.t[2]); break;
      case MPK_OP_TENSOR_INIT: add(outs, l.t[0]); break;
      case MPK_OP_QUANTIZE_FP8: add(ins, l.t[0]); add(outs, l.t[1]); add(outs, l.t[2]); break;
      case MPK_OP_LINEAR_FP8: for (int i = 0; i < 4; ++i) add(ins, l.t[i]); add(outs, l.t[4]); break;
      case MPK_OP_MOE_TOPK_SIGMOID:
        add(ins, l.t[0]); add(ins, l.t[1]); add(outs, l.t[0]); add(outs, l.t[2]); add(outs, l.t[3]); add(outs, l.t[4]); break;
      case MPK_OP_MOE_TOPK_SOFTMAX:
        add(ins, l.t[0]); add(outs, l.t[1]); add(outs, l.t[2]); add(outs, l.t[3]); break;
      case MPK_OP_MOE_W13_LINEAR: case MPK_OP_MOE_W2_LINEAR:
        for (int i = 0; i < 4; ++i) add(ins, l.t[i]); add(outs, l.t[4]); break;
      case MPK_OP_MOE_W13_FP8: case MPK_OP_MOE_W2_FP8:
        for (int i = 0; i < 6; ++i) add(ins, l.t[i]); add(outs, l.t[6]); break;
      case MPK_OP_MOE_SILU_MUL: add(ins, l.t[0]); add(outs, l.t[1]); break;
      case MPK_OP_MOE_MUL_SUM_ADD: add(ins, l.t[0]); add(ins, l.t[1]); add(ins, l.t[2]); add(outs, l.t[3]); break;
      case MPK_OP_MLA_KV_GATHER: add(ins, l.t[0]); add(ins, l.t[1]); add(ins, l.t[2]); add(outs, l.t[2]); break;
      case MPK_OP_MLA_DECODE: add(ins, l.t[0]); add(ins, l.t[1]); add(outs, l.t[2]); add(outs, l.t[3]); break;
      case MPK_OP_MLA_REDUCE: add(ins, l.t[0]); add(ins, l.t[1]); add(outs, l.t[2]); break;
      case MPK_OP_LINEAR_FP8_RESIDUAL: for (int i = 0; i < 5; ++i) add(ins, l.t[i]); add(outs, l.t[5]); break;
      default: break;
    }
  }

  bool raw_reads(const LayerInfo &l, int storage) const {
    // does the un-folded layer read this storage?
    std::vector<int> ins, outs;
    layer_io(l, &ins, &outs);
    for (int t : ins) if (T[t].storage == storage) return true;
    return false;
  }
  bool raw_writes(const LayerInfo &l, int storage) const {
    std::vector<int> ins, outs;
    layer_io(l, &ins, &outs);
    for (int t : outs) if (T[t].storage == storage) return true;
    return false;
  }

  int check_arity() {
    for (size_t i = 0; i < L.size(); ++i) {
      static const std::map<int, int> need = {
          {MPK_OP_EMBED, 3}, {MPK_OP_RMSNORM, 3}, {MPK_OP_RMSNORM_LINEAR, 4}, {MPK_OP_LINEAR, 3},
          {MPK_OP_LINEAR_RESIDUAL, 4}, {MPK_OP_SPLITK_LINEAR, 3}, {MPK_OP_ATTENTION, 8},
          {MPK_OP_PAGED_ATTENTION, 8}, {MPK_OP_SILU_MUL, 2}, {MPK_OP_ALLREDUCE, 3},
          {MPK_OP_ARGMAX_PARTIAL, 3}, {MPK_OP_ARGMAX_REDUCE, 3}, {MPK_OP_ELEMENTWISE_ADD, 3},
          {MPK_OP_TENSOR_INIT, 1}, {MPK_OP_QUANTIZE_FP8, 3}, {MPK_OP_LINEAR_FP8, 5}, {MPK_OP_LINEAR_FP8_RESIDUAL, 6},
          {MPK_OP_MOE_TOPK_SIGMOID, 5}, {MPK_OP_MOE_W13_LINEAR, 5}, {MPK_OP_MOE_W2_LINEAR, 5}, {MPK_OP_MOE_W13_FP8, 7},
          {MPK_OP_MOE_W2_FP8, 7}, {MPK_OP_MOE_SILU_MUL, 2}, {MPK_OP_MOE_MUL_SUM_ADD, 4},
          {MPK_OP_MLA_KV_GATHER, 3}, {MPK_OP_MLA_DECODE, 4}, {MPK_OP_MLA_REDUCE, 3},
          {MPK_OP_SAMPLING_PARTIAL, 3}, {MPK_OP_SAMPLING_REDUCE, 3}, {MPK_OP_ARGMAX_EXCHANGE, 3},
          {MPK_OP_MOE_TOPK_SOFTMAX, 4}};
      auto it = need.find(L[i].op);
      if (it == need.end()) return fail(MPK_ERR_UNSUPPORTED, "layer " + std::to_string(i) + ": unknown op");
      if ((int)L[i].t.size() < it->second)
        return fail(MPK_ERR_INVALID, "layer " + std::to_string(i) + ": expected " + std::to_string(it->second) +
                                         " tensors");
      for (int t : L[i].t)
        if (t >= (int)T.size()) return fail(MPK_ERR_INVALID, "layer " + std::to_string(i) + ": bad tensor id");
    }
    return MPK_OK;
  }

  // ---- folding ----------------------------------------------------------------
  void fold_layers() {
    // RMSNORM_LINEAR is a linear with a norm prologue from the start.
    for (auto &l : L)
      if (l.op == MPK_OP_RMSNORM_LINEAR) {
        LayerInfo n = l;
        n.op = MPK_OP_LINEAR;
        n.t = {l.t[0], l.t[2], l.t[3]};
        n.prologue = PRO_RMSNORM;
        n.pro_src = l.t[0];
        n.pro_gamma = l.t[1];
        l = n;
      }
    for (size_t i = 0; i < L.size(); ++i) {
      LayerInfo &p = L[i];
      if (p.folded || (p.op != MPK_OP_RMSNORM && p.op != MPK_OP_SILU_MUL)) continue;
      const int y = p.op == MPK_OP_RMSNORM ? p.t[2] : p.t[1];
      const int src = p.t[0];
      if (T[y].owner == 0) continue;   // caller-visible buffer: keep it materialised
      std::vector<size_t> consumers;
      bool ok = true;
      for (size_t j = i + 1; j < L.size() && ok; ++j) {
        const LayerInfo &c = L[j];
        const bool reads = raw_reads(c, T[y].storage);
        if (reads) {
          const bool lin = (c.op == MPK_OP_LINEAR || c.op == MPK_OP_LINEAR_RESIDUAL ||
                            c.op == MPK_OP_SPLITK_LINEAR) && c.prologue == PRO_PLAIN && c.t[0] == y;
          // y must not also be this consumer's residual / accumulate operand
          const bool other_use = (c.op == MPK_OP_LINEAR_RESIDUAL && T[c.t[2]].storage == T[y].storage);
          if (!lin || other_use) ok = false;
          else consumers.push_back(j);
          // the norm prologue needs the whole row in the activation tile
          if (ok && p.op == MPK_OP_RMSNORM && linear_tile_bytes(T[c.t[1]].dim(1)) > x_tile_cap()) ok = false;
        }
        if (raw_writes(c, T[y].storage)) break;           // y redefined: later readers see the new value
      }
      if (!ok || consumers.empty()) continue;
      // no layer between the producer and its last consumer may overwrite the source
      for (size_t j = i + 1; j < consumers.back() && ok; ++j)
        if (raw_writes(L[j], T[src].storage)) ok = false;
      if (!ok) continue;
      for (size_t j : consumers) {
        LayerInfo &c = L[j];
        if (p.op == MPK_OP_RMSNORM) {
          c.prologue = PRO_RMSNORM;
          c.pro_src = src;
          c.pro_gamma = p.t[1];
        } else {
          c.prologue = PRO_SILU_MUL;
          c.pro_src = src;
          c.pro_groups = std::max(p.grid[0], 1);
        }
      }
      p.folded = true;
      g->num_folded++;
    }
  }

  // ---- allreduce fusion: linear -> allreduce becomes push epilogue + reduce tasks -----
  int plan_allreduce() {
    auto pushing_linear = [&](int j) {
      return j >= 0 && (L[j].op == MPK_OP_LINEAR || L[j].op == MPK_OP_LINEAR_RESIDUAL || L[j].op == MPK_OP_SPLITK_LINEAR);
    };
    auto producer_of = [&](size_t i) {
      for (int j = (int)i - 1; j >= 0; --j)
        if (!L[j].folded && raw_writes(L[j], T[L[i].t[0]].storage)) return j;
      return -1;
    };
    // An allreduce whose input comes from anything but a bf16 linear (an FP8 linear, the weighted sum of a
    // mixture-of-experts block, ...) gets a push stage of its own in front of it: the input is materialised by its
    // producer as usual and copied into the ranks' inboxes by TASK_AR_PUSH tasks.
    for (size_t i = 0; i < L.size(); ++i) {
      if (L[i].op != MPK_OP_ALLREDUCE) continue;
      if (cfg.world_size <= 1) return fail(MPK_ERR_INVALID, "allreduce_layer with world_size 1");
      const int prod = producer_of(i);
      if (prod < 0) return fail(MPK_ERR_UNSUPPORTED, "allreduce input is not produced inside the graph");
      if (pushing_linear(prod)) continue;
      if (T[L[i].t[0]].dtype != MPK_BF16 || T[L[i].t[0]].dims.size() != 2)
        return fail(MPK_ERR_UNSUPPORTED, "allreduce input must be a 2-D bf16 tensor");
      LayerInfo p;
      p.op = MPK_OP_AR_PUSH;
      p.t = {L[i].t[0]};
      L.insert(L.begin() + i, p);
      ++i;
    }
    int idx = 0;
    for (size_t i = 0; i < L.size(); ++i) {
      LayerInfo &a = L[i];
      if (a.op != MPK_OP_ALLREDUCE) continue;
      const int x = a.t[0];
      int prod = (i > 0 && L[i - 1].op == MPK_OP_AR_PUSH && L[i - 1].t[0] == x) ? (int)i - 1 : producer_of(i);
      if (prod < 0 || !(pushing_linear(prod) || L[prod].op == MPK_OP_AR_PUSH))
        return fail(MPK_ERR_UNSUPPORTED, "allreduce input must be produced by a linear layer");
      for (size_t j = prod + 1; j < L.size(); ++j) {
        if (j != i && !L[j].folded && raw_reads(L[j], T[x].storage) && j < i)
          return fail(MPK_ERR_UNSUPPORTED, "allreduce input has another reader before the allreduce");
      }
      L[prod].push = true;
      L[prod].ar_index = idx;
      a.ar_producer = prod;
      a.ar_index = idx++;
    }
    // an argmax exchange is one more instance in the same sequence (its words live in their own area of the inbox)
    for (auto &a : L)
      if (a.op == MPK_OP_ARGMAX_EXCHANGE) {
        if (cfg.world_size <= 1) return fail(MPK_ERR_INVALID, "argmax exchange with world_size 1");
        a.ar_index = idx++;
      }
    g->num_allreduce = idx;
    fold_allreduce();
    return MPK_OK;
  }

  // Fold an allreduce into the linears that consume its result: the producer pushes self-validating words,
  // the consumers' prologue gathers, reduces, adds the residual and materialises the tensor.  No task and
  // no event remain for the allreduce itself.
  void fold_allreduce() {
    // Only for graphs of at most 8 batched tokens.  The fused form makes EVERY consumer CTA poll and read the whole
    // [world][tokens][K] inbox: 8 KB per rank at one token, but 128 KB per rank at 16 -- at 8 ranks 148 CTAs pulling
    // 2 MB each per allreduce, measured at 12.2 ms per 16-token step on 8 GPUs against 6.0 ms on one.  With more
    // tokens the allreduce stays a task group of its own: fp32 partials pushed by the producer's epilogue, summed once
    // by reduce tasks spread over the workers, read as an ordinary activation by the consumers.
    if (cfg.max_num_batched_tokens > 8) return;
    auto is_lin = [](int op) { return op == MPK_OP_LINEAR || op == MPK_OP_LINEAR_RESIDUAL || op == MPK_OP_SPLITK_LINEAR; };
    for (size_t i = 0; i < L.size(); ++i) {
      LayerInfo &a = L[i];
      if (a.op != MPK_OP_ALLREDUCE || a.ar_producer < 0) continue;
      if (L[a.ar_producer].op == MPK_OP_AR_PUSH) continue;   // (fp32 slots + remote event: summed by TASK_ALLREDUCE)
      LayerInfo &prod = L[a.ar_producer];
      const int y = a.t[2];
      const int res = (prod.op == MPK_OP_LINEAR_RESIDUAL || prod.op == MPK_OP_SPLITK_LINEAR) ? prod.t[2] : -1;
      if (T[y].dims.size() != 2 || T[y].dtype != MPK_BF16) continue;
      std::vector<size_t> consumers;
      bool ok = true;
      for (size_t j = i + 1; j < L.size() && ok; ++j) {
        const LayerInfo &c = L[j];
        if (c.folded) continue;
        if (raw_reads(c, T[y].storage)) {
          const bool as_input = is_lin(c.op) && c.gather_ar < 0 &&
                                ((c.prologue == PRO_RMSNORM && c.pro_src == y) || (c.prologue == PRO_PLAIN && c.t[0] == y)) &&
                                T[c.t[1]].dim(1) == T[y].dim(1);
          const bool as_pushed_residual = is_lin(c.op) && c.push && c.t[2] == y && !as_input &&
                                          !(c.prologue == PRO_PLAIN && c.t[0] == y) && c.pro_src != y;
          const bool as_ar_residual = c.op == MPK_OP_ALLREDUCE;
          if (as_input) consumers.push_back(j);
          else if (!as_pushed_residual && !as_ar_residual) ok = false;
        }
        if (j != i && raw_writes(c, T[y].storage)) break;
      }
      if (!ok || consumers.empty()) continue;
      for (size_t j : consumers) {
        L[j].gather_ar = a.ar_index;
        L[j].gather_res = res;
        L[j].gather_out = y;
      }
      prod.push_ll = true;
      a.folded = true;
      g->num_folded++;
    }
  }

  // ---- shared-memory plan ---------------------------------------------------------
  int plan_smem() {
    const int ntok = std::min(std::max(cfg.max_num_batched_tokens, 1), (int)kMaxLinearTokens);
    int64_t need = 24 * 1024;
    for (const auto &l : L) {
      if (l.folded) continue;
      if (l.op == MPK_OP_LINEAR || l.op == MPK_OP_LINEAR_RESIDUAL || l.op == MPK_OP_SPLITK_LINEAR) {
        const int64_t K = T[l.t[1]].dim(1);
        need = std::max(need, std::min<int64_t>(linear_tile_bytes(K), x_tile_cap()));
        if (tc_linear(K) && T[l.t[1]].dtype == MPK_BF16) g->use_tmem = true;
      } else if (l.op == MPK_OP_LINEAR_FP8 || l.op == MPK_OP_LINEAR_FP8_RESIDUAL) {
        const int64_t K = T[l.t[2]].dim(1);
        if (tc_linear_fp8(K)) {
          g->use_tmem = true;
          int64_t KT = K;
          while (KT > 512 && (fp8_tc_tile_bytes(KT) - kPartialBytes > fp8_tc_tile_cap() || K % KT != 0 || KT % 512 != 0)) KT -= 512;
          need = std::max<int64_t>(need, fp8_tc_tile_bytes(KT) - kPartialBytes);
        } else {
          need = std::max(need, std::min<int64_t>(fp8_tile_bytes(ntok, K), x_tile_cap()));
        }
      } else if (l.op == MPK_OP_MOE_W13_FP8 || l.op == MPK_OP_MOE_W2_FP8) {
        need = std::max(need, std::min<int64_t>(moe_fp8_tile_bytes(ntok, T[l.t[2]].dim(2)), x_tile_cap()));
      } else if (l.op == MPK_OP_MOE_W13_LINEAR || l.op == MPK_OP_MOE_W2_LINEAR) {
        need = std::max(need, std::min<int64_t>((int64_t)ntok * (T[l.t[1]].dim(2) * 2 + kRowPadBytes), x_tile_cap()));
      } else if (l.op == MPK_OP_MLA_DECODE) {
        need = std::max<int64_t>(need, 16 * (576 * 2 + 16) + 64 * (576 * 2 + 16) + 16 * (64 * 2 + 16) + 2 * 8 * 16 * 4);
      } else if (l.op == MPK_OP_MOE_TOPK_SIGMOID) {
        const int64_t E = T[l.t[0]].dim(1);
        need = std::max(need, 8 * (2 * E + 64) * 4 + E * 4 + 64);
      } else if (l.op == MPK_OP_ATTENTION || l.op == MPK_OP_PAGED_ATTENTION) {
        const int G = (int)(l.params[0] / l.params[1]);
        int64_t attn = (int64_t)G * (128 + 16 + 8 * 128) * 4 + (int64_t)cfg.max_num_batched_tokens * 512;
        // the general instantiation streams cached K/V rows through 32 KB stages (two at least) beside the query
        // heads, the per-warp maxima / sums, 256 page ids and the rows of the new tokens
        if (general_graph()) {
          const int64_t new_rows = (std::min(cfg.max_num_batched_tokens, 64) + 7) / 8 * 8;
          attn = 8 * 272 + (int64_t)G * 64 + 1024 + 2 * new_rows * 272 + 2 * (8 * 2 * 8 * 272);   // two stages per warp
        }
        need = std::max(need, attn - kPartialBytes);
      }
    }
    if (!no_batch_task()) need = std::max<int64_t>(need, (int64_t)(13 * cfg.max_num_batched_requests + 16) * 4 - kPartialBytes);
    need = (need + 255) / 256 * 256;
    // 64 KB stages (4 KB row segments) when at least three of them fit, else 32 KB stages
    const int64_t room = kSmemBudget - kMiscBytesHost - kPartialBytes - need;
    g->x_tile_bytes = (int)need;
    g->tc_tokens = tc_np();
    if (g->use_tmem) {
      // tcgen05 graphs: a ring of 16 KB slots (whole swizzle atoms), each filled by one tensor-map TMA; tasks that
      // still stream padded rows (FP8, expert projections) take the widest chunk such a slot holds
      const int stages = (int)(room / kTcSlotBytes);
      if (stages < 2) return fail(MPK_ERR_UNSUPPORTED, "activation tile leaves fewer than 2 weight stages");
      g->stage_bytes = kTcSlotBytes;
      g->chunk_cols = 448;                 // 16 rows x (448 x 2 + 16) bytes <= 16 KB
      g->num_stages = std::min(stages, 8);
      return MPK_OK;
    }
    int cols = kChunkColsMax;
    if (room / stage_bytes_for(cols) < (nb_max <= 8 ? 3 : 2)) cols = kChunkColsMax / 2;
    const int stages = (int)(room / stage_bytes_for(cols));
    if (stages < 2) return fail(MPK_ERR_UNSUPPORTED, "activation tile leaves fewer than 2 weight stages");
    g->chunk_cols = cols;
    g->stage_bytes = stage_bytes_for(cols);
    g->num_stages = std::min(stages, 8);   // (the kernel uses the upper half of its 16-entry barrier arrays as scratch)
    return MPK_OK;
  }

  // ---- task emission ----------------------------------------------------------------
  TaskDesc blank(uint32_t type, int layer) {
    TaskDesc d;
    std::memset(&d, 0, sizeof(d));
    d.type = type;
    d.layer = layer;
    for (int i = 0; i < kMaxDeps; ++i) d.dep_event[i] = -1;
    d.trig_event = -1;
    return d;
  }
  void put(int worker, const TaskDesc &d, int exec) {
    per_worker[worker].push_back(d);
    per_worker_exec[worker].push_back(exec);
    g->exec[exec].num_tasks++;
  }

  int emit_linear(int li, int ex) {
    const LayerInfo &l = L[li];
    const TensorInfo &w = T[l.t[1]];
    const int yid = l.op == MPK_OP_LINEAR_RESIDUAL ? l.t[3] : l.t[2];
    const TensorInfo &y = T[yid];
    if (w.dims.size() != 2 || w.dtype != MPK_BF16)
      return fail(MPK_ERR_UNSUPPORTED, "linear weight must be a 2-D bf16 tensor: " + w.name);
    if (w.strides[1] != 1) return fail(MPK_ERR_UNSUPPORTED, "linear weight must be row-major: " + w.name);
    const int N = (int)w.dim(0), K = (int)w.dim(1), ldw = (int)w.strides[0];
    if (cfg.max_num_batched_tokens > kMaxLinearTokens)
      return fail(MPK_ERR_UNSUPPORTED, "linear layers support at most 64 batched tokens in this build");
    if (K % 16 != 0 || ldw % 8 != 0) return fail(MPK_ERR_UNSUPPORTED, "linear K must be a multiple of 16: " + w.name);
    // k tiling of the activation tile: the fewest tiles whose [tokens, KT] slab fits the tile buffer
    const int ntok = std::min(std::max(cfg.max_num_batched_tokens, 1), (int)kMaxLinearTokens);
    const bool tc = g->use_tmem && tc_linear(K);
    const int kq = tc ? kTcKBlock : 16;   // granularity of a k tile
    int nkt = 1;
    while (nkt <= K / kq &&
           !(K % nkt == 0 && (K / nkt) % kq == 0 && linear_tile_bytes(K / nkt) <= g->x_tile_bytes))
      ++nkt;
    if (nkt > K / kq) return fail(MPK_ERR_UNSUPPORTED, "cannot tile K for " + w.name);
    const int KT = K / nkt;
    if (l.prologue == PRO_RMSNORM && nkt != 1)
      return fail(MPK_ERR_UNSUPPORTED, "rmsnorm prologue needs the whole row in shared memory: " + w.name);
    // k extent of a streamed chunk: the largest multiple of 16 that divides KT and fits a stage
    // Chunk geometry: 16 rows (one mma m-tile) x KC columns.  The copy engine handles a fixed number of bulk
    // copies per unit time, so row segments should be long: KC is as wide as the stage allows.
    const int R = kChunkRows;
    int KC = std::min(KT, g->chunk_cols) / 16 * 16;
    while (KC > 16 && KT % KC != 0) KC -= 16;
    // with several k tiles the partial sums of a task wait in shared memory: two row groups at most
    const int cap = nkt > 1 ? 2 * R : (1 << 20);
    // source of the activation
    const int xsrc = l.prologue == PRO_PLAIN ? l.t[0] : l.pro_src;
    const TensorInfo &x = T[xsrc];
    if (l.prologue == PRO_SILU_MUL) {
      if (x.dim(1) != 2 * (int64_t)K || (K / l.pro_groups) % 8 != 0 || K % l.pro_groups != 0)
        return fail(MPK_ERR_INVALID, "silu_mul feeding " + w.name + ": bad gate|up width or group count");
    } else if (x.dim(x.dims.size() - 1) != K) {
      return fail(MPK_ERR_INVALID, "linear input width != K for " + w.name);
    }
    if (y.dim(y.dims.size() - 1) != N) return fail(MPK_ERR_INVALID, "linear output width != N for " + w.name);
    int epi = EPI_STORE;
    uint64_t res_ptr = 0;
    int ldr = 0;
    if (l.op == MPK_OP_LINEAR_RESIDUAL) {
      const bool enable = l.params.empty() ? true : l.params[0] != 0;
      // With tensor parallelism the reference adds the residual on rank 0 only
      // (python/mirage/mpk/persistent_kernel.py:1783-1787); here the residual of a pushed
      // linear is added once by the reduce tasks instead, on every rank identically.
      if (enable && !l.push) { epi = EPI_RESIDUAL; res_ptr = (uint64_t)T[l.t[2]].ptr; ldr = (int)T[l.t[2]].ld(); }
    } else if (l.op == MPK_OP_SPLITK_LINEAR && !l.push) {
      epi = EPI_RESIDUAL; res_ptr = (uint64_t)y.ptr; ldr = (int)y.ld();
    }
    if (l.push) epi = l.push_ll ? EPI_PUSH_LL : EPI_PUSH_F32;
    uint64_t out_ptr = (uint64_t)y.ptr;
    int ldo = (int)y.ld();
    const int unit = l.silu_out >= 0 ? 4 : 1;      // paired rows stay in one task
    if (l.silu_out >= 0) {
      if (epi != EPI_STORE || N % 4 != 0) return fail(MPK_ERR_INVALID, "activation epilogue on an unsupported linear: " + w.name);
      epi = EPI_SILU_PAIR;
      out_ptr = (uint64_t)T[l.silu_out].ptr;
      ldo = (int)T[l.silu_out].ld();
    }
    bool w_dynamic = false;
    for (const auto &o : L) if (!o.folded && raw_writes(o, w.storage)) w_dynamic = true;
    const int base = (N / unit) / W, rem = (N / unit) % W;
    // tcgen05 path: cut the widest worker panel into row tiles of RB <= 128 rows (one accumulator each) and give a
    // ring slot as many 64-column k blocks of such a tile as it holds; among the tilings near the minimum, take
    // the one that fills the slots best (the bytes in flight per worker are what hides the HBM latency)
    int tc_rb = 0, tc_nkb = 1, tc_task_rows = 0;
    if (tc) {
      const int cnt_max = (base + (rem ? 1 : 0)) * unit;
      const int kbt = KT / kTcKBlock;
      const int t_min = (cnt_max + 127) / 128;
      // Measured: an M = 128 bf16 tcgen05.mma with N <= 64 occupies the tensor pipe for about 43 cycles whatever N is
      // and however few of its 128 rows are real, and a worker must consume ~23 weight bytes per cycle to keep up
      // with its share of HBM.  A K = 16 step of a tile with r real rows consumes 32 r bytes: r must exceed ~31
      // for the MMAs to stay ahead of the stream, so tiles keep at least 40 real rows where the panel allows.
      const int need_rows = 40;
      double best = -1.0;
      for (int tiles = t_min; tiles <= t_min + 6; ++tiles) {
        const int rb = ((cnt_max + tiles - 1) / tiles + 7) / 8 * 8;
        if (rb > 128 || rb <= 0) continue;
        if (tiles > t_min && cnt_max / tiles < need_rows) break;
        int nkb = std::min(kbt, g->stage_bytes / (rb * 128));
        while (nkb > 1 && kbt % nkb != 0) --nkb;
        if (nkb < 1) continue;
        const double fill = (double)cnt_max / tiles * 128.0 * nkb / g->stage_bytes;
        if (fill > best * 1.05) { best = fill; tc_rb = rb; tc_nkb = nkb; }
      }
      if (tc_rb == 0) return fail(MPK_ERR_UNSUPPORTED, "cannot tile the rows of " + w.name);
      tc_task_rows = std::max(1, kTcAccCols / tc_np()) * tc_rb;   // accumulators of one task: tiles x tc_np() columns
      g->exec[ex].tc_rows = tc_rb;
      g->exec[ex].tc_kblocks = tc_nkb;
    }
    const int task_cap = tc ? tc_task_rows : cap;
    int row = 0;
    for (int i = 0; i < W; ++i) {
      const int worker = (i + rot) % W;
      const int cnt = (base + (i < rem ? 1 : 0)) * unit;
      bool first = true;
      for (int r = row; r < row + cnt; r += task_cap) {
        TaskDesc d = blank(TASK_LINEAR, li);
        if (!first && nkt == 1) d.flags |= TF_SAME_X_AS_PREV;
        if (w_dynamic) d.flags |= TF_STREAM_AFTER_DEP;
        d.p[0] = (uint64_t)w.ptr;
        d.p[1] = (uint64_t)x.ptr;
        d.p[2] = out_ptr;
        d.p[3] = res_ptr;
        d.p[4] = l.prologue == PRO_RMSNORM ? (uint64_t)T[l.pro_gamma].ptr : 0;
        d.p[5] = in.inbox_base_floats;
        if (l.gather_ar >= 0) {
          d.p[6] = l.gather_res >= 0 ? (uint64_t)T[l.gather_res].ptr : 0;
          d.p[7] = (uint64_t)T[l.gather_out].ptr;
          d.a[L_GATHER] = l.gather_ar + 1;
          d.a[L_G_LDRES] = l.gather_res >= 0 ? (int)T[l.gather_res].ld() : 0;
          d.a[L_G_LDOUT] = (int)T[l.gather_out].ld();
          d.a[L_G_SLOT] = cfg.max_num_batched_tokens * K;
        }
        d.a[L_N0] = r;
        d.a[L_N1] = std::min(r + task_cap, row + cnt);
        d.a[L_K] = K;
        d.a[L_LDW] = ldw;
        d.a[L_LDX] = (int)x.ld();
        d.a[L_LDO] = ldo;
        d.a[L_LDR] = ldr;
        d.a[L_PRO] = l.prologue;
        d.a[L_EPI] = epi;
        d.a[L_EPS] = float_bits(1e-6f);
        d.a[L_GROUPS] = l.pro_groups;
        d.a[L_KT] = KT;
        d.a[L_KC] = KC;
        d.a[L_ROWS] = R;
        d.a[L_SLOT] = cfg.max_num_batched_tokens * N;
        d.a[L_N] = N;
        d.a[L_ARIDX] = std::max(l.ar_index, 0);
        d.a[L_NAR] = g->num_allreduce;
        d.a[L_PARSTRIDE] = (int)g->inbox_floats_per_buffer;
        if (tc) {
          d.flags |= TF_TC;
          d.a[L_KC] = tc_nkb * kTcKBlock;
          d.a[L_ROWS] = tc_rb;
          d.a[L_TMAP] = (int)g->tmaps.size();
          TmapSpec m;
          m.base = (uint64_t)w.ptr + (uint64_t)r * (uint64_t)ldw * 2;
          m.rows = d.a[L_N1] - d.a[L_N0];
          m.ld_bytes = (int64_t)ldw * 2;
          m.kblocks = K / kTcKBlock;
          m.box_rows = tc_rb;
          m.box_kblocks = tc_nkb;
          m.elt_bytes = 2;
          g->tmaps.push_back(m);
        }
        put(worker, d, ex);
        g->weight_bytes += (int64_t)(d.a[L_N1] - d.a[L_N0]) * K * 2;
        first = false;
      }
      row += cnt;
    }
    return MPK_OK;
  }

  // Strides (in uint32 words) of a packed UE8M0 scale tensor over (outer index, packed k).  Accepted layouts:
  // logical [outer, packed_k] with any strides, or the physical column-major form [packed_k, aligned_outer]
  // that the reference's builders allocate (python/mirage/mpk/models/deepseek_v3/builder.py:166-174).
  int ue8m0_strides(const TensorInfo &s, int64_t outer, int64_t pk, bool activation, int *s_outer, int *s_pk) {
    if (s.dims.size() != 2 || (s.dtype != MPK_U32 && s.dtype != MPK_I32))
      return fail(MPK_ERR_INVALID, "packed UE8M0 scales must be a 2-D uint32 tensor: " + s.name);
    const bool logical = s.dim(0) >= outer && s.dim(1) == pk;
    const bool physical = s.dim(0) == pk && s.dim(1) >= outer;
    if (!logical && !physical)
      return fail(MPK_ERR_INVALID, "scale tensor " + s.name + " matches neither [outer, K/512] nor [K/512, outer]");
    // a square tensor fits both readings: activation scales are then taken in the physical form the
    // reference's quantiser writes, weight scales in the logical form its checkpoints converters attach
    if (physical && (!logical || activation)) {
      *s_outer = (int)s.strides[1]; *s_pk = (int)s.strides[0];
    } else {
      *s_outer = (int)s.strides[0]; *s_pk = (int)s.strides[1];
    }
    return MPK_OK;
  }

  // FP8 linear: e4m3 weights [N, K] and activations [tokens, K], UE8M0 scales per 128 columns of each row
  // (python/mirage/mpk/persistent_kernel.py:1584-1632).  Same streaming geometry as the bf16 linear with one
  // byte per element; a task covers at most kFp8TaskRows weight rows so that their scales fit in the tile.
  int emit_linear_fp8(int li, int ex) {
    const LayerInfo &l = L[li];
    const bool has_res = l.op == MPK_OP_LINEAR_FP8_RESIDUAL;
    const TensorInfo &x = T[l.t[0]], &xs = T[l.t[1]], &w = T[l.t[2]], &ws = T[l.t[3]];
    const TensorInfo &y = T[l.t[has_res ? 5 : 4]];
    if (w.dims.size() != 2 || w.dtype != MPK_F8E4M3 || x.dtype != MPK_F8E4M3 || w.strides[1] != 1)
      return fail(MPK_ERR_UNSUPPORTED, "linear_fp8 needs row-major 2-D e4m3 weight and activations: " + w.name);
    const int N = (int)w.dim(0), K = (int)w.dim(1), ldw = (int)w.strides[0];
    if (K % 128 != 0 || ldw % 16 != 0) return fail(MPK_ERR_UNSUPPORTED, "linear_fp8 K must be a multiple of 128: " + w.name);
    if (x.dim(x.dims.size() - 1) != K || x.ld() % 16 != 0) return fail(MPK_ERR_INVALID, "linear_fp8 input width != K for " + w.name);
    if (y.dim(y.dims.size() - 1) != N || y.dtype != MPK_BF16) return fail(MPK_ERR_INVALID, "linear_fp8 output must be bf16 [tokens, N]: " + w.name);
    if (cfg.max_num_batched_tokens > kMaxLinearTokens)
      return fail(MPK_ERR_UNSUPPORTED, "linear layers support at most 64 batched tokens in this build");
    const int64_t pk = (K / 128 + 3) / 4;
    int ws0, ws1, xs0, xs1;
    int rc = ue8m0_strides(ws, N, pk, false, &ws0, &ws1);
    if (rc) return rc;
    rc = ue8m0_strides(xs, cfg.max_num_batched_tokens, pk, true, &xs0, &xs1);
    if (rc) return rc;
    const int ntok = std::min(std::max(cfg.max_num_batched_tokens, 1), (int)kMaxLinearTokens);
    const bool tc = g->use_tmem && tc_linear_fp8(K);
    int nkt = 1;
    if (tc) {
      while (nkt <= K / 512 && !(K % nkt == 0 && (K / nkt) % 512 == 0 && fp8_tc_tile_bytes(K / nkt) <= g->x_tile_bytes + kPartialBytes)) ++nkt;
      if (nkt > K / 512) return fail(MPK_ERR_UNSUPPORTED, "cannot tile K for " + w.name);
    } else {
      while (nkt <= K / 128 && !(K % nkt == 0 && (K / nkt) % 128 == 0 && fp8_tile_bytes(ntok, K / nkt) <= g->x_tile_bytes)) ++nkt;
      if (nkt > K / 128) return fail(MPK_ERR_UNSUPPORTED, "cannot tile K for " + w.name);
    }
    const int KT = K / nkt;
    const int R = kChunkRows;
    int KC = std::min(KT, g->chunk_cols * 2) / 128 * 128;   // a stage holds twice as many one-byte columns
    while (KC > 128 && KT % KC != 0) KC -= 128;
    int cap = nkt > 1 ? 2 * R : kFp8TaskRows;
    bool w_dynamic = false;
    for (const auto &o : L) if (!o.folded && raw_writes(o, w.storage)) w_dynamic = true;
    const bool enable_res = has_res && (l.params.empty() || l.params[0] != 0);
    const int base = N / W, rem = N % W;
    // tcgen05 path: row tiles and k blocks per ring slot chosen as for the bf16 linears (a k block is 128 one-byte
    // columns); a task holds at most kTcFp8MaxTiles tiles
    int tc_rb = 0, tc_nkb = 1;
    if (tc) {
      const int cnt_max = base + (rem ? 1 : 0);
      const int kbt = KT / 128;
      const int t_min = (cnt_max + 127) / 128;
      double best = -1.0;
      for (int tiles = t_min; tiles <= t_min + 6; ++tiles) {
        const int rb = ((cnt_max + tiles - 1) / tiles + 7) / 8 * 8;
        if (rb > 128 || rb <= 0) continue;
        if (tiles > t_min && cnt_max / tiles < 40) break;
        int nkb = std::min(kbt, g->stage_bytes / (rb * 128));
        while (nkb > 1 && kbt % nkb != 0) --nkb;
        if (nkb < 1) continue;
        const double fill = (double)cnt_max / tiles * 128.0 * nkb / g->stage_bytes;
        if (fill > best * 1.05) { best = fill; tc_rb = rb; tc_nkb = nkb; }
      }
      if (tc_rb == 0) return fail(MPK_ERR_UNSUPPORTED, "cannot tile the rows of " + w.name);
      cap = std::min<int>(kTcFp8MaxTiles, std::max(1, kTcAccCols / tc_np())) * tc_rb;
      KC = tc_nkb * 128;
      g->exec[ex].tc_rows = tc_rb;
      g->exec[ex].tc_kblocks = tc_nkb;
    }
    int row = 0;
    for (int i = 0; i < W; ++i) {
      const int worker = (i + rot) % W;
      const int cnt = base + (i < rem ? 1 : 0);
      bool first = true;
      for (int r = row; r < row + cnt; r += cap) {
        TaskDesc d = blank(TASK_LINEAR, li);
        d.flags |= TF_FP8;
        if (!first && nkt == 1) d.flags |= TF_SAME_X_AS_PREV;
        if (w_dynamic) d.flags |= TF_STREAM_AFTER_DEP;
        d.p[0] = (uint64_t)w.ptr;
        d.p[1] = (uint64_t)x.ptr;
        d.p[2] = (uint64_t)y.ptr;
        d.p[3] = enable_res ? (uint64_t)T[l.t[4]].ptr : 0;
        d.p[6] = (uint64_t)ws.ptr;
        d.p[7] = (uint64_t)xs.ptr;
        d.a[L_N0] = r;
        d.a[L_N1] = std::min(r + cap, row + cnt);
        d.a[L_K] = K;
        d.a[L_LDW] = ldw;
        d.a[L_LDX] = (int)x.ld();
        d.a[L_LDO] = (int)y.ld();
        d.a[L_LDR] = enable_res ? (int)T[l.t[4]].ld() : 0;
        d.a[L_PRO] = PRO_PLAIN;
        d.a[L_EPI] = enable_res ? EPI_RESIDUAL : EPI_STORE;
        d.a[L_KT] = KT;
        d.a[L_KC] = KC;
        d.a[L_ROWS] = R;
        d.a[L_N] = N;
        d.a[L_WS_S0] = ws0; d.a[L_WS_S1] = ws1; d.a[L_XS_S0] = xs0; d.a[L_XS_S1] = xs1;
        if (tc) {
          d.flags |= TF_TC;
          d.a[L_ROWS] = tc_rb;
          d.a[L_TMAP] = (int)g->tmaps.size();
          TmapSpec m;
          m.base = (uint64_t)w.ptr + (uint64_t)r * (uint64_t)ldw;
          m.rows = d.a[L_N1] - d.a[L_N0];
          m.ld_bytes = ldw;
          m.kblocks = K / 128;
          m.box_rows = tc_rb;
          m.box_kblocks = tc_nkb;
          m.elt_bytes = 1;
          g->tmaps.push_back(m);
        }
        put(worker, d, ex);
        g->weight_bytes += (int64_t)(d.a[L_N1] - d.a[L_N0]) * K;
        first = false;
      }
      row += cnt;
    }
    return MPK_OK;
  }

  // Per-token, per-128-column quantisation to e4m3 (python/mirage/mpk/persistent_kernel.py:1561-1582):
  // a task takes a range of tokens and a range of 512-column packs.
  int emit_quantize_fp8(int li, int ex) {
    const LayerInfo &l = L[li];
    const TensorInfo &x = T[l.t[0]], &q = T[l.t[1]], &s = T[l.t[2]];
    const bool ue8m0 = l.params.empty() || l.params[0] != 0;
    if (x.dtype != MPK_BF16 || q.dtype != MPK_F8E4M3) return fail(MPK_ERR_INVALID, "quantize_fp8: bf16 in, e4m3 out");
    const int nd = (int)x.dims.size();
    const int64_t K = x.dim(nd - 1);
    int64_t rows = 1;
    for (int i = 0; i < nd - 1; ++i) rows *= x.dim(i);
    if (K % 128 != 0) return fail(MPK_ERR_UNSUPPORTED, "quantize_fp8 width must be a multiple of 128");
    if (x.strides[nd - 1] != 1 || q.strides[nd - 1] != 1 || (nd > 2 && (x.strides[nd - 2] != K || q.strides[nd - 2] != K)))
      return fail(MPK_ERR_UNSUPPORTED, "quantize_fp8 tensors must be dense in their leading dimensions");
    const int64_t ng = K / 128, pk = (ng + 3) / 4;
    int s0, s1;
    if (ue8m0) {
      if (nd != 2) return fail(MPK_ERR_UNSUPPORTED, "quantize_fp8 with packed scales takes 2-D tensors");
      const int rc = ue8m0_strides(s, rows, pk, true, &s0, &s1);
      if (rc) return rc;
    } else {
      if (s.dtype != MPK_F32 || (int64_t)(s.bytes / 4) < rows * ng) return fail(MPK_ERR_INVALID, "quantize_fp8 float32 scales must be [rows, K/128]");
      s0 = (int)ng; s1 = 1;
    }
    // tokens: with a 2-D input only the active tokens are quantised; higher-rank inputs (token x expert) are
    // treated as rows of the flattened tensor
    const int per_tok = (int)(rows / std::max<int64_t>(x.dim(0), 1));
    const int nt = (int)std::max<int64_t>(1, std::min<int64_t>(W, rows * pk));
    const int64_t units = rows * pk;
    for (int i = 0; i < nt; ++i) {
      TaskDesc d = blank(TASK_QUANTIZE_FP8, li);
      d.p[0] = (uint64_t)x.ptr; d.p[1] = (uint64_t)q.ptr; d.p[2] = (uint64_t)s.ptr;
      d.a[0] = (int)(units * i / nt); d.a[1] = (int)(units * (i + 1) / nt);   // (row, pack) units
      d.a[2] = (int)K; d.a[3] = (int)(nd == 2 ? x.strides[0] : K); d.a[4] = (int)(nd == 2 ? q.strides[0] : K);
      d.a[5] = ue8m0 ? 1 : 0; d.a[6] = per_tok; d.a[7] = s0; d.a[8] = s1; d.a[9] = (int)pk;
      put((i + rot) % W, d, ex);
    }
    return MPK_OK;
  }

  // Expert projections (python/mirage/mpk/persistent_kernel.py:1444-1559, 1652-1681): every worker owns a row
  // range of EVERY expert and walks the list of active experts at run time, so the work is balanced whatever the
  // routing; a worker with more rows than a task may hold gets several tasks.
  int emit_moe_gemm(int li, int ex) {
    const LayerInfo &l = L[li];
    const bool fp8 = l.op == MPK_OP_MOE_W13_FP8 || l.op == MPK_OP_MOE_W2_FP8;
    const bool w2 = l.op == MPK_OP_MOE_W2_LINEAR || l.op == MPK_OP_MOE_W2_FP8;
    const TensorInfo &x = T[l.t[0]], &w = T[l.t[fp8 ? 2 : 1]], &idx = T[l.t[fp8 ? 4 : 2]], &mask = T[l.t[fp8 ? 5 : 3]];
    const TensorInfo &y = T[l.t[fp8 ? 6 : 4]];
    if (w.dims.size() != 3 || y.dims.size() != 3 || (int)x.dims.size() != (w2 ? 3 : 2))
      return fail(MPK_ERR_INVALID, "expert projection: weight [E, N, K], output [B, topk, N]: " + w.name);
    // E counts the experts of the routing tensors; the weight tensor may hold a contiguous range of them starting at
    // params[0] (expert parallelism): experts outside never reach the active list, so addressing a virtual expert 0
    // params[0] panels below the tensor is enough
    const int E = (int)idx.dim(0), EW = (int)w.dim(0), ebase = l.params.empty() ? 0 : (int)l.params[0];
    const int N = (int)w.dim(1), K = (int)w.dim(2), topk = (int)y.dim(1);
    if (ebase < 0 || ebase + EW > E) return fail(MPK_ERR_INVALID, "expert projection: weight experts outside the routing range: " + w.name);
    const int want = fp8 ? MPK_F8E4M3 : MPK_BF16;
    if (w.dtype != want || x.dtype != want || y.dtype != MPK_BF16 || w.strides[2] != 1 || w.strides[1] != K ||
        w.strides[0] != (int64_t)N * K)
      return fail(MPK_ERR_UNSUPPORTED, "expert projection: dense " + std::string(fp8 ? "e4m3" : "bf16") + " weights, bf16 output: " + w.name);
    if (x.dim(x.dims.size() - 1) != K || y.dim(2) != N || mask.dim(0) != E + 1 || idx.dtype != MPK_I32 ||
        mask.dtype != MPK_I32 || (w2 && x.dim(1) != topk) || topk > 255 || idx.dim(1) > 255)
      return fail(MPK_ERR_INVALID, "expert projection: shapes of " + w.name + " and its routing tensors disagree");
    if (K % 128 != 0 || (int64_t)N * K >= (1ll << 31))
      return fail(MPK_ERR_UNSUPPORTED, "expert projection: K must be a multiple of 128: " + w.name);
    if ((((uint64_t)x.ptr | (uint64_t)w.ptr) & 15u) != 0)     // rows are gathered / streamed with 16-byte copies
      return fail(MPK_ERR_UNSUPPORTED, "expert projection: input and weight must start on a 16-byte boundary: " + w.name);
    if (cfg.max_num_batched_tokens > kMaxLinearTokens)
      return fail(MPK_ERR_UNSUPPORTED, "linear layers support at most 64 batched tokens in this build");
    if (fp8) {
      const TensorInfo &xs = T[l.t[1]], &ws = T[l.t[3]];
      if (xs.dtype != MPK_F32 || ws.dtype != MPK_F32 || (int64_t)(ws.bytes / 4) < (int64_t)EW * N * (K / 128) ||
          xs.dim(xs.dims.size() - 1) != K / 128)
        return fail(MPK_ERR_INVALID, "expert projection: float32 scales [.., K/128] expected: " + w.name);
      // the task copies scales four at a time (16-byte asynchronous copies) when a row holds a multiple of four
      if ((K / 128) % 4 == 0 && (((uint64_t)xs.ptr | (uint64_t)ws.ptr) & 15u) != 0)
        return fail(MPK_ERR_UNSUPPORTED, "expert projection: scale tensors must start on a 16-byte boundary: " + w.name);
    }
    const int ntok = std::min(std::max(cfg.max_num_batched_tokens, 1), (int)kMaxLinearTokens);
    auto tile_bytes = [&](int KT) { return fp8 ? moe_fp8_tile_bytes(ntok, KT) : (int64_t)ntok * (KT * 2 + kRowPadBytes); };
    int nkt = 1;
    while (nkt <= K / 128 && !(K % nkt == 0 && (K / nkt) % 128 == 0 && tile_bytes(K / nkt) <= g->x_tile_bytes)) ++nkt;
    if (nkt > K / 128) return fail(MPK_ERR_UNSUPPORTED, "cannot tile K for " + w.name);
    const int KT = K / nkt;
    const int R = kChunkRows;
    const int step = fp8 ? 128 : 64;
    int KC = std::min(KT, g->chunk_cols * (fp8 ? 2 : 1)) / step * step;
    while (KC > step && KT % KC != 0) KC -= step;
    const int cap = nkt > 1 ? 2 * R : kFp8TaskRows;
    const int base = N / W, rem = N % W;
    int row = 0;
    for (int i = 0; i < W; ++i) {
      const int worker = (i + rot) % W;
      const int cnt = base + (i < rem ? 1 : 0);
      for (int r = row; r < row + cnt; r += cap) {
        TaskDesc d = blank(TASK_MOE_GEMM, li);
        d.flags |= TF_STREAM_AFTER_DEP | (fp8 ? TF_FP8 : 0u);
        d.p[0] = (uint64_t)w.ptr - (uint64_t)ebase * (uint64_t)N * K * (fp8 ? 1 : 2);
        d.p[1] = (uint64_t)x.ptr; d.p[2] = (uint64_t)y.ptr;
        d.p[4] = (uint64_t)idx.ptr; d.p[5] = (uint64_t)mask.ptr;
        if (fp8) {
          d.p[6] = (uint64_t)T[l.t[3]].ptr - (uint64_t)ebase * (uint64_t)N * (K / 128) * 4;
          d.p[7] = (uint64_t)T[l.t[1]].ptr;
        }
        d.a[L_N0] = r; d.a[L_N1] = std::min(r + cap, row + cnt); d.a[L_K] = K; d.a[L_LDW] = K; d.a[L_LDX] = K;
        d.a[L_LDO] = N; d.a[L_KT] = KT; d.a[L_KC] = KC; d.a[L_ROWS] = R; d.a[L_N] = N;
        d.a[M_NEXP] = E; d.a[M_NTOPK] = topk; d.a[M_PER_SLOT] = w2 ? 1 : 0; d.a[M_LDR] = (int)idx.dim(1);
        d.a[M_ESTRIDE] = N * K;
        put(worker, d, ex);
      }
      row += cnt;
    }
    return MPK_OK;
  }

  int emit_attention(int li, int ex, int attn_ordinal) {
    const LayerInfo &l = L[li];
    const bool paged = l.op == MPK_OP_PAGED_ATTENTION;
    if (l.params.size() < 4) return fail(MPK_ERR_INVALID, "attention needs [hq, hkv, qk_norm, rope] params");
    const int hq = (int)l.params[0], hkv = (int)l.params[1];
    const int qk_norm = (int)l.params[2], rope = (int)l.params[3];
    const TensorInfo &kc = T[l.t[1]];
    if (kc.dims.size() != 4 || kc.dim(3) != 128)
      return fail(MPK_ERR_UNSUPPORTED, "attention supports head_dim 128 caches [pages|batch, page|seq, kv_heads, 128]");
    if (hkv <= 0 || hq % hkv != 0) return fail(MPK_ERR_INVALID, "q heads must be a multiple of kv heads");
    const int G = hq / hkv;
    if (G != 1 && G != 2 && G != 4 && G != 8) return fail(MPK_ERR_UNSUPPORTED, "GQA group size must be 1, 2, 4 or 8");
    if (kc.dim(2) != hkv) return fail(MPK_ERR_INVALID, "kv cache head count != num_kv_heads");
    if (!cfg.qo_indptr && paged && !cfg.dry_run) return fail(MPK_ERR_INVALID, "paged attention needs the batch meta tensors");
    const int slots = paged ? cfg.max_num_batched_requests : std::max(l.grid[0], 1);
    const int page = paged ? (int)kc.dim(1) : (int)kc.dim(1);
    if (paged && page != cfg.page_size) return fail(MPK_ERR_INVALID, "kv cache page size != page_size");
    if (paged && general_graph() && page % 8 != 0)
      return fail(MPK_ERR_UNSUPPORTED, "with more than 8 batched tokens (or FP8 / expert layers) the page size must be a multiple of 8");
    const int max_seq = paged ? cfg.max_seq_length : (int)kc.dim(1);
    // chunks per (request, kv head): enough to give every worker a task, and with many requests enough that a
    // task stays near 128 rows at full length (the rows a task prefetches before its dependency wait are its
    // cheapest ones; long serial chunks are latency-bound)
    int NC = std::max(1, W / std::max(slots * hkv, 1));
    if (general_graph()) {
      // streamed K/V: long chunks are cheap (a task's fixed part is paid once), so a (request, kv head) pair is cut
      // only as far as it takes to occupy the workers, and into chunks of at most ~2048 positions so that requests
      // of very different lengths still spread evenly
      NC = std::max(NC, (max_seq + 2047) / 2048);
    } else {
      NC = std::max(NC, std::min((max_seq + 127) / 128, 16));
    }
    NC = std::min(NC, std::max(1, max_seq / 32));
    NC = std::min(NC, 32);
    const int rope_rows = rope ? (int)T[l.t[5]].dim(0) : 1;
    for (int s = 0; s < slots; ++s)
      for (int h = 0; h < hkv; ++h)
        for (int c = 0; c < NC; ++c) {
          TaskDesc d = blank(TASK_ATTENTION, li);
          for (int i = 0; i < 8; ++i) d.p[i] = l.t[i] >= 0 ? (uint64_t)T[l.t[i]].ptr : 0;
          d.a[A_SLOT] = s;
          d.a[A_HEAD] = h;
          d.a[A_CHUNK] = c;
          d.a[A_NCHUNK] = NC;
          d.a[A_HQ] = hq;
          d.a[A_HKV] = hkv;
          d.a[A_HD] = 128;
          d.a[A_PAGE] = page;
          d.a[A_FLAGS] = (qk_norm ? 1 : 0) | (rope ? 2 : 0) | (paged ? 0 : 4);
          d.a[A_LDQKV] = (int)T[l.t[0]].ld();
          d.a[A_LDO] = (int)T[l.t[7]].ld();
          d.a[A_EPS] = float_bits(1e-6f);
          d.a[A_ROPE_ROWS] = rope_rows;
          d.a[A_CSEQ] = (int)kc.dim(1);
          d.a[A_TICKET] = attn_ordinal;   // ticket bank
          d.a[A_EARLY_EV] = no_batch_task() ? -1 : 0;   // exec layer 0 is the batching task
          d.a[A_EARLY_NEED] = 1;
          put(((s * hkv + h) * NC + c + rot) % W, d, ex);
        }
    g->attn_scratch_floats =
        std::max<int64_t>(g->attn_scratch_floats, (int64_t)cfg.max_num_batched_tokens * hq * NC * 130);
    g->attn_tickets = std::max<int64_t>(g->attn_tickets, (int64_t)slots * hkv);
    return MPK_OK;
  }

  void emit_token_rows(uint32_t type, int li, int ex, uint64_t p0, uint64_t p1, uint64_t p2, int width, int ldi,
                       int ldo, int aux, int ldi2, int rows_total) {
    const int nt = std::min(rows_total, W);
    for (int i = 0; i < nt; ++i) {
      TaskDesc d = blank(type, li);
      d.p[0] = p0; d.p[1] = p1; d.p[2] = p2;
      d.a[E_T0] = (int)((int64_t)rows_total * i / nt);
      d.a[E_T1] = (int)((int64_t)rows_total * (i + 1) / nt);
      d.a[E_WIDTH] = width; d.a[E_LDI] = ldi; d.a[E_LDO] = ldo; d.a[E_AUX] = aux; d.a[E_LDI2] = ldi2;
      put((i + rot) % W, d, ex);
    }
  }

  int emit(int li, int ex, int *attn_ordinal) {
    const LayerInfo &l = L[li];
    const int mbt = cfg.max_num_batched_tokens;
    switch (l.op) {
      case MPK_OP_LINEAR: case MPK_OP_LINEAR_RESIDUAL: case MPK_OP_SPLITK_LINEAR:
        return emit_linear(li, ex);
      case MPK_OP_LINEAR_FP8: case MPK_OP_LINEAR_FP8_RESIDUAL:
        return emit_linear_fp8(li, ex);
      case MPK_OP_QUANTIZE_FP8:
        return emit_quantize_fp8(li, ex);
      case MPK_OP_MOE_W13_LINEAR: case MPK_OP_MOE_W2_LINEAR: case MPK_OP_MOE_W13_FP8: case MPK_OP_MOE_W2_FP8:
        return emit_moe_gemm(li, ex);
      case MPK_OP_MOE_TOPK_SOFTMAX: {
        // the same task as the sigmoid routing with one group, no bias and scaling 1: only the score function differs
        const TensorInfo &lg = T[l.t[0]], &w = T[l.t[1]], &idx = T[l.t[2]], &mask = T[l.t[3]];
        const int E = (int)lg.dim(1), topk = (int)w.dim(1);
        if ((lg.dtype != MPK_BF16 && lg.dtype != MPK_F32) || w.dtype != MPK_F32 || idx.dtype != MPK_I32 || mask.dtype != MPK_I32 ||
            E > 1024 || idx.dim(0) != E || mask.dim(0) != E + 1 || topk <= 0 || topk > std::min(E, 32) || idx.dim(1) > kMaxLinearTokens)
          return fail(MPK_ERR_UNSUPPORTED, "softmax routing: logits bf16/f32 [B, E <= 1024], weights f32 [B, topk <= 32], indices and mask int32");
        TaskDesc d = blank(TASK_MOE_ROUTING, li);
        d.p[0] = (uint64_t)lg.ptr; d.p[1] = 0; d.p[2] = (uint64_t)w.ptr; d.p[3] = (uint64_t)idx.ptr; d.p[4] = (uint64_t)mask.ptr;
        d.a[0] = E; d.a[1] = topk; d.a[2] = 1; d.a[3] = 1; d.a[4] = float_bits(1.0f); d.a[5] = (int)lg.ld();
        d.a[6] = (int)w.ld(); d.a[7] = (int)idx.dim(1); d.a[8] = lg.dtype == MPK_F32 ? 1 : 0;
        d.a[9] = l.params.size() > 1 ? (int)l.params[0] : 0;
        d.a[10] = l.params.size() > 1 ? (int)l.params[1] : E;
        d.a[11] = 1;   // softmax scores, logits left in place
        if (d.a[9] < 0 || d.a[10] > E || d.a[9] >= d.a[10]) return fail(MPK_ERR_INVALID, "softmax routing: bad local expert range");
        put(rot % W, d, ex);
        return MPK_OK;
      }
      case MPK_OP_MOE_TOPK_SIGMOID: {
        const TensorInfo &lg = T[l.t[0]], &bias = T[l.t[1]], &w = T[l.t[2]], &idx = T[l.t[3]], &mask = T[l.t[4]];
        if (l.params.size() < 3) return fail(MPK_ERR_INVALID, "sigmoid routing needs [num_groups, topk_group, scaling_bits]");
        const int E = (int)lg.dim(1), topk = (int)w.dim(1), groups = (int)l.params[0], keep = (int)l.params[1];
        if ((lg.dtype != MPK_BF16 && lg.dtype != MPK_F32) || bias.dtype != MPK_F32 || w.dtype != MPK_F32 ||
            idx.dtype != MPK_I32 || mask.dtype != MPK_I32)
          return fail(MPK_ERR_INVALID, "sigmoid routing: logits bf16/f32, bias and weights f32, indices and mask int32");
        if (groups <= 0 || groups > 64 || E % groups != 0 || keep <= 0 || keep > groups || E > 1024 || bias.dim(0) != E ||
            idx.dim(0) != E || mask.dim(0) != E + 1 || topk <= 0 || topk > keep * (E / groups) || idx.dim(1) > kMaxLinearTokens)
          return fail(MPK_ERR_UNSUPPORTED, "sigmoid routing: unsupported expert / group / top-k configuration");
        TaskDesc d = blank(TASK_MOE_ROUTING, li);
        d.p[0] = (uint64_t)lg.ptr; d.p[1] = (uint64_t)bias.ptr; d.p[2] = (uint64_t)w.ptr; d.p[3] = (uint64_t)idx.ptr;
        d.p[4] = (uint64_t)mask.ptr;
        d.a[0] = E; d.a[1] = topk; d.a[2] = groups; d.a[3] = keep; d.a[4] = (int)l.params[2]; d.a[5] = (int)lg.ld();
        d.a[6] = (int)w.ld(); d.a[7] = (int)idx.dim(1); d.a[8] = lg.dtype == MPK_F32 ? 1 : 0;
        // optional params [3], [4]: first and one-past-last expert this rank runs (expert parallelism)
        d.a[9] = l.params.size() > 4 ? (int)l.params[3] : 0;
        d.a[10] = l.params.size() > 4 ? (int)l.params[4] : E;
        if (d.a[9] < 0 || d.a[10] > E || d.a[9] >= d.a[10] || topk > 32)
          return fail(MPK_ERR_INVALID, "sigmoid routing: bad local expert range");
        put(rot % W, d, ex);
        return MPK_OK;
      }
      case MPK_OP_MLA_KV_GATHER: {
        const TensorInfo &lat = T[l.t[0]], &pe = T[l.t[1]], &cache = T[l.t[2]];
        if (l.params.size() < 3) return fail(MPK_ERR_INVALID, "mla_kv_gather needs [d_k, d_v, page_size]");
        const int dk = (int)l.params[0], dv = (int)l.params[1], page = (int)l.params[2];
        if (dk != 576 || dv != 512 || cache.dims.size() != 3 || cache.dim(1) != page || cache.dim(2) != dk ||
            lat.dtype != MPK_BF16 || pe.dtype != MPK_BF16 || cache.dtype != MPK_BF16 || lat.dim(1) < dv || pe.dim(1) < dk - dv)
          return fail(MPK_ERR_UNSUPPORTED, "mla_kv_gather: bf16 cache [pages, page, 576], c_latent [tokens, 512], k_pe [tokens, >= 64]");
        if (!cfg.qo_indptr || !cfg.paged_kv_indptr || !cfg.paged_kv_indices || !cfg.paged_kv_last_page_len) {
          if (!cfg.dry_run) return fail(MPK_ERR_INVALID, "mla_kv_gather needs the batch meta tensors");
        }
        for (int s = 0; s < cfg.max_num_batched_requests; ++s) {
          TaskDesc d = blank(TASK_MLA_APPEND, li);
          d.p[0] = (uint64_t)lat.ptr; d.p[1] = (uint64_t)pe.ptr; d.p[2] = (uint64_t)cache.ptr;
          d.a[0] = s; d.a[1] = (int)lat.ld(); d.a[2] = (int)pe.ld(); d.a[3] = page; d.a[4] = dk; d.a[5] = dv;
          put((s + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      case MPK_OP_MLA_DECODE: {
        const TensorInfo &q = T[l.t[0]], &cache = T[l.t[1]], &po = T[l.t[2]], &lse = T[l.t[3]];
        if (l.params.size() < 6) return fail(MPK_ERR_INVALID, "mla decode needs [heads, q_len, kv_len, splits, scale, page]");
        const int H = (int)l.params[0], q_len = (int)l.params[1], kv_len = (int)l.params[2], S = (int)l.params[3];
        const int page = (int)l.params[5];
        if (H <= 0 || H % 16 != 0 || q.dim(q.dims.size() - 1) != (int64_t)H * 576 || q.dtype != MPK_BF16 ||
            cache.dtype != MPK_BF16 || po.dtype != MPK_BF16 || lse.dtype != MPK_F32 || S != (kv_len + 127) / 128)
          return fail(MPK_ERR_UNSUPPORTED, "mla decode: bf16 q [tokens, heads * 576] with heads a multiple of 16");
        if ((int64_t)(po.bytes / 2) < (int64_t)mbt * H * S * 512 || (int64_t)(lse.bytes / 4) < (int64_t)mbt * H * S)
          return fail(MPK_ERR_INVALID, "mla decode: partial buffers hold fewer than tokens x heads x splits rows");
        if (page > 0 && (cache.dims.size() != 3 || cache.dim(1) != page || cache.dim(2) != 576))
          return fail(MPK_ERR_INVALID, "mla decode: paged cache must be [pages, page, 576]");
        if (page > 0 && !cfg.dry_run && (!cfg.qo_indptr || !cfg.paged_kv_indptr || !cfg.paged_kv_indices || !cfg.paged_kv_last_page_len))
          return fail(MPK_ERR_INVALID, "mla decode on a paged cache needs the batch meta tensors");
        if (page == 0 && (q_len <= 0 || mbt % q_len != 0 || (int64_t)(cache.bytes / 2) < (int64_t)(mbt / q_len) * kv_len * 576))
          return fail(MPK_ERR_INVALID, "mla decode: dense cache must be [requests * kv_len, 576] with q_len tokens per request");
        int i = 0;
        for (int t = 0; t < mbt; ++t)
          for (int s = 0; s < S; ++s)
            for (int h0 = 0; h0 < H; h0 += 16, ++i) {
              TaskDesc d = blank(TASK_MLA_DECODE, li);
              d.p[0] = (uint64_t)q.ptr; d.p[1] = (uint64_t)cache.ptr; d.p[2] = (uint64_t)po.ptr; d.p[3] = (uint64_t)lse.ptr;
              d.a[0] = t; d.a[1] = s; d.a[2] = h0; d.a[3] = H; d.a[4] = S; d.a[5] = page; d.a[6] = (int)q.ld();
              d.a[7] = (int)l.params[4]; d.a[8] = q_len; d.a[9] = kv_len;
              put((i + rot) % W, d, ex);
            }
        return MPK_OK;
      }
      case MPK_OP_MLA_REDUCE: {
        const TensorInfo &po = T[l.t[0]], &lse = T[l.t[1]], &y = T[l.t[2]];
        if (l.params.size() < 2) return fail(MPK_ERR_INVALID, "mla reduce needs [heads, splits]");
        const int H = (int)l.params[0], S = (int)l.params[1];
        if (S > 64) return fail(MPK_ERR_UNSUPPORTED, "mla reduce handles at most 64 splits (8192 positions)");
        if (y.dtype != MPK_BF16 || (int64_t)(y.bytes / 2) < (int64_t)mbt * H * 512 || po.dtype != MPK_BF16 || lse.dtype != MPK_F32)
          return fail(MPK_ERR_INVALID, "mla reduce: bf16 output [tokens, heads * 512]");
        const int rows = mbt * H, nt = std::max(1, std::min(W, rows / 8));
        for (int i = 0; i < nt; ++i) {
          TaskDesc d = blank(TASK_MLA_REDUCE, li);
          d.p[0] = (uint64_t)po.ptr; d.p[1] = (uint64_t)lse.ptr; d.p[2] = (uint64_t)y.ptr;
          d.a[0] = (int)((int64_t)rows * i / nt); d.a[1] = (int)((int64_t)rows * (i + 1) / nt); d.a[2] = H; d.a[3] = S;
          d.a[4] = y.dims.size() == 2 ? (int)y.ld() : H * 512;
          put((i + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      case MPK_OP_MOE_SILU_MUL: {
        const TensorInfo &m = T[l.t[0]], &y = T[l.t[1]];
        if (m.dims.size() != 3 || y.dims.size() != 3 || m.dim(2) != 2 * y.dim(2) || m.dtype != MPK_BF16)
          return fail(MPK_ERR_INVALID, "moe_silu_mul: [B, topk, 2I] -> [B, topk, I] bf16");
        const int rows = (int)(y.dim(0) * y.dim(1)), nt = std::min(rows, W);
        for (int i = 0; i < nt; ++i) {
          TaskDesc d = blank(TASK_MOE_SILU_MUL, li);
          d.p[0] = (uint64_t)m.ptr; d.p[2] = (uint64_t)y.ptr;
          d.a[0] = (int)((int64_t)rows * i / nt); d.a[1] = (int)((int64_t)rows * (i + 1) / nt);
          d.a[2] = (int)y.dim(2); d.a[3] = (int)m.strides[1]; d.a[4] = (int)y.strides[1]; d.a[5] = (int)y.dim(1);
          put((i + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      case MPK_OP_MOE_MUL_SUM_ADD: {
        const TensorInfo &x = T[l.t[0]], &w = T[l.t[1]], &y = T[l.t[3]];
        const bool has_res = l.t[2] >= 0;
        if (x.dims.size() != 3 || w.dtype != MPK_F32 || x.dtype != MPK_BF16 || y.dim(1) != x.dim(2) || w.dim(1) != x.dim(1))
          return fail(MPK_ERR_INVALID, "moe_mul_sum_add: x [B, topk, H] bf16, weights [B, topk] f32, out [B, H]");
        const int H = (int)x.dim(2), nt = std::max(1, std::min(W, H / 64));
        for (int i = 0; i < nt; ++i) {
          TaskDesc d = blank(TASK_MOE_MUL_SUM_ADD, li);
          d.p[0] = (uint64_t)x.ptr; d.p[1] = (uint64_t)w.ptr; d.p[2] = (uint64_t)y.ptr;
          d.p[3] = has_res ? (uint64_t)T[l.t[2]].ptr : 0;
          d.a[0] = (int)((int64_t)H * i / nt); d.a[1] = (int)((int64_t)H * (i + 1) / nt); d.a[2] = H; d.a[3] = (int)x.dim(1);
          d.a[4] = (int)y.ld(); d.a[5] = has_res ? (int)T[l.t[2]].ld() : 0; d.a[6] = (int)w.ld(); d.a[7] = (int)x.dim(0);
          put((i + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      case MPK_OP_ATTENTION: case MPK_OP_PAGED_ATTENTION:
        return emit_attention(li, ex, (*attn_ordinal)++);
      case MPK_OP_EMBED: {
        const TensorInfo &tab = T[l.t[1]], &y = T[l.t[2]];
        if (T[l.t[0]].dtype != MPK_I64) return fail(MPK_ERR_INVALID, "embed ids must be int64");
        if (tab.dim(1) % 8 != 0) return fail(MPK_ERR_UNSUPPORTED, "embedding width must be a multiple of 8");
        emit_token_rows(TASK_EMBED, li, ex, (uint64_t)T[l.t[0]].ptr, (uint64_t)tab.ptr, (uint64_t)y.ptr,
                        (int)tab.dim(1), (int)tab.ld(), (int)y.ld(), (int)tab.dim(0), 0, mbt);
        return MPK_OK;
      }
      case MPK_OP_RMSNORM: {
        const TensorInfo &x = T[l.t[0]], &y = T[l.t[2]];
        if (x.dim(1) % 8 != 0) return fail(MPK_ERR_UNSUPPORTED, "rmsnorm width must be a multiple of 8");
        emit_token_rows(TASK_RMSNORM, li, ex, (uint64_t)x.ptr, (uint64_t)T[l.t[1]].ptr, (uint64_t)y.ptr,
                        (int)x.dim(1), (int)x.ld(), (int)y.ld(), float_bits(1e-6f), 0, (int)std::min<int64_t>(x.dim(0), mbt));
        return MPK_OK;
      }
      case MPK_OP_ELEMENTWISE_ADD: {
        const TensorInfo &a = T[l.t[0]], &b = T[l.t[1]], &y = T[l.t[2]];
        emit_token_rows(TASK_ELEMENTWISE_ADD, li, ex, (uint64_t)a.ptr, (uint64_t)b.ptr, (uint64_t)y.ptr,
                        (int)a.dim(1), (int)a.ld(), (int)y.ld(), 0, (int)b.ld(), (int)std::min<int64_t>(a.dim(0), mbt));
        return MPK_OK;
      }
      case MPK_OP_TENSOR_INIT: {
        const TensorInfo &t = T[l.t[0]];
        const int es = elt_size(t.dtype);
        const int rows = (int)t.dim(0);
        const int64_t row_bytes = (int64_t)(t.bytes / std::max(rows, 1));
        if (row_bytes % 4 != 0) return fail(MPK_ERR_UNSUPPORTED, "tensor_init rows must be a multiple of 4 bytes");
        (void)es;
        emit_token_rows(TASK_TENSOR_INIT, li, ex, 0, 0, (uint64_t)t.ptr, (int)row_bytes, 0, (int)row_bytes, 0, 0, rows);
        return MPK_OK;
      }
      case MPK_OP_SILU_MUL: {
        const TensorInfo &m = T[l.t[0]], &y = T[l.t[1]];
        const int I = (int)y.dim(1);
        const int groups = std::max(l.grid[0], 1);
        if (m.dim(1) != 2 * (int64_t)I || I % groups != 0) return fail(MPK_ERR_INVALID, "silu_mul shapes");
        // column ranges in units of 8 (one 16-byte vector); about 4096 elements of work per task at least
        const int units = I % 8 == 0 ? I / 8 : I, unit = I % 8 == 0 ? 8 : 1;
        const int nt = (int)std::max<int64_t>(1, std::min<int64_t>({(int64_t)W, (int64_t)units, (int64_t)mbt * I / 4096}));
        for (int i = 0; i < nt; ++i) {
          TaskDesc d = blank(TASK_SILU_MUL, li);
          d.p[0] = (uint64_t)m.ptr; d.p[2] = (uint64_t)y.ptr;
          d.a[E_T0] = 0; d.a[E_T1] = mbt; d.a[E_WIDTH] = I; d.a[E_LDI] = (int)m.ld(); d.a[E_LDO] = (int)y.ld();
          d.a[E_AUX] = groups;
          d.a[7] = (int)((int64_t)units * i / nt) * unit;
          d.a[8] = (int)((int64_t)units * (i + 1) / nt) * unit;
          put((i + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      case MPK_OP_ARGMAX_PARTIAL: case MPK_OP_SAMPLING_PARTIAL: {
        const TensorInfo &lg = T[l.t[0]], &pv = T[l.t[1]], &pi = T[l.t[2]];
        const bool sampling = l.op == MPK_OP_SAMPLING_PARTIAL;
        const int n = std::max(l.grid[0], 1);
        const int V = (int)lg.dim(1);
        if (pv.dim(1) < n || pi.dim(1) < n || pi.dtype != MPK_I64)
          return fail(MPK_ERR_INVALID, "argmax partial buffers must be [tokens, >= grid.x], index int64");
        for (int i = 0; i < n; ++i) {
          TaskDesc d = blank(sampling ? TASK_SAMPLING_PARTIAL : TASK_ARGMAX_PARTIAL, li);
          d.p[0] = (uint64_t)lg.ptr; d.p[1] = (uint64_t)pv.ptr; d.p[2] = (uint64_t)pi.ptr;
          d.a[0] = (int)((int64_t)V * i / n); d.a[1] = (int)((int64_t)V * (i + 1) / n); d.a[2] = i;
          d.a[3] = (int)lg.ld(); d.a[4] = (int)pv.ld();
          if (sampling) {   // Gumbel-max: philox seed and the rows one reference task would see (noise repeats per task)
            const uint64_t seed = l.params.size() > 0 ? (uint64_t)l.params[0] : 42u;
            d.a[6] = (int)(uint32_t)seed; d.a[7] = (int)(uint32_t)(seed >> 32);
            d.a[8] = l.params.size() > 1 ? std::max((int)l.params[1], 1) : 1;
            d.a[9] = V;
          }
          put((i + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      case MPK_OP_ARGMAX_REDUCE: case MPK_OP_SAMPLING_REDUCE: {
        const TensorInfo &pv = T[l.t[0]], &pi = T[l.t[1]], &o = T[l.t[2]];
        const int partial_op = l.op == MPK_OP_SAMPLING_REDUCE ? MPK_OP_SAMPLING_PARTIAL : MPK_OP_ARGMAX_PARTIAL;
        if (o.dtype != MPK_I64) return fail(MPK_ERR_INVALID, "argmax output must be int64");
        // number of partials = tasks of the producing partial layer
        int n = (int)pv.dim(1);
        for (int j = li - 1; j >= 0; --j)
          if (L[j].op == partial_op && T[L[j].t[1]].storage == pv.storage) { n = std::max(L[j].grid[0], 1); break; }
        TaskDesc d = blank(l.op == MPK_OP_SAMPLING_REDUCE ? TASK_SAMPLING_REDUCE : TASK_ARGMAX_REDUCE, li);
        d.p[0] = (uint64_t)pv.ptr; d.p[1] = (uint64_t)pi.ptr; d.p[2] = (uint64_t)o.ptr;
        d.a[0] = n; d.a[1] = (int)pv.ld();
        put(rot % W, d, ex);
        return MPK_OK;
      }
      case MPK_OP_ARGMAX_EXCHANGE: {
        const TensorInfo &pv = T[l.t[0]], &pi = T[l.t[1]], &o = T[l.t[2]];
        if (o.dtype != MPK_I64 || pi.dtype != MPK_I64) return fail(MPK_ERR_INVALID, "argmax output and indices must be int64");
        int n = (int)pv.dim(1);
        for (int j = li - 1; j >= 0; --j)
          if (L[j].op == MPK_OP_ARGMAX_PARTIAL && T[L[j].t[1]].storage == pv.storage) { n = std::max(L[j].grid[0], 1); break; }
        TaskDesc d = blank(TASK_ARGMAX_EXCHANGE, li);
        d.p[0] = (uint64_t)pv.ptr; d.p[1] = (uint64_t)pi.ptr; d.p[2] = (uint64_t)o.ptr;
        d.p[5] = in.inbox_base_floats + (uint64_t)exchange_base_words;
        d.a[0] = n; d.a[1] = (int)pv.ld();
        d.a[2] = l.params.empty() ? 0 : (int)l.params[0];
        d.a[L_ARIDX] = l.ar_index;
        d.a[L_NAR] = g->num_allreduce;
        d.a[L_PARSTRIDE] = (int)g->inbox_floats_per_buffer;
        put(rot % W, d, ex);
        return MPK_OK;
      }
      case MPK_OP_AR_PUSH: {
        const TensorInfo &x = T[l.t[0]];
        const int N = (int)x.dim(1);
        const int nt = std::max(1, std::min(W, N / 64));
        for (int i = 0; i < nt; ++i) {
          TaskDesc d = blank(TASK_AR_PUSH, li);
          d.p[0] = (uint64_t)x.ptr; d.p[5] = in.inbox_base_floats;
          d.a[0] = (int)((int64_t)N * i / nt); d.a[1] = (int)((int64_t)N * (i + 1) / nt);
          d.a[2] = (int)x.ld(); d.a[3] = mbt * N; d.a[6] = N;
          d.a[7] = l.ar_index; d.a[8] = g->num_allreduce; d.a[9] = (int)g->inbox_floats_per_buffer;
          put((i + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      case MPK_OP_ALLREDUCE: {
        const LayerInfo &p = L[l.ar_producer];
        const TensorInfo &y = T[l.t[2]];
        const int N = (int)y.dim(1);
        const int nt = std::max(1, std::min(W, N / 64));
        uint64_t res = 0; int ldr = 0;
        if (p.op == MPK_OP_LINEAR_RESIDUAL) { res = (uint64_t)T[p.t[2]].ptr; ldr = (int)T[p.t[2]].ld(); }
        if (p.op == MPK_OP_SPLITK_LINEAR) { res = (uint64_t)T[p.t[2]].ptr; ldr = (int)T[p.t[2]].ld(); }
        for (int i = 0; i < nt; ++i) {
          TaskDesc d = blank(TASK_ALLREDUCE, li);
          d.p[0] = in.inbox_base_floats; d.p[1] = res; d.p[2] = (uint64_t)y.ptr;
          d.a[0] = (int)((int64_t)N * i / nt); d.a[1] = (int)((int64_t)N * (i + 1) / nt);
          d.a[2] = cfg.world_size; d.a[3] = mbt * N; d.a[4] = (int)y.ld(); d.a[5] = ldr; d.a[6] = N;
          d.a[7] = l.ar_index; d.a[8] = g->num_allreduce; d.a[9] = (int)g->inbox_floats_per_buffer;
          put((i + rot) % W, d, ex);
        }
        return MPK_OK;
      }
      default: return fail(MPK_ERR_UNSUPPORTED, "op not implemented");
    }
  }

  int run() {
    int rc = check_arity();
    if (rc) return rc;
    for (const auto &l : L) if (l.folded) g->num_folded++;     // folded before materialisation (activation epilogue)
    fold_layers();
    rc = plan_allreduce();
    if (rc) return rc;
    rc = plan_smem();
    if (rc) return rc;
    // inbox sizing: widest pushed output
    int64_t nmax = 0;
    for (const auto &l : L)
      if (l.push) nmax = std::max<int64_t>(nmax, l.op == MPK_OP_AR_PUSH ? T[l.t[0]].dim(1) : T[l.t[1]].dim(0));
    g->inbox_floats_per_buffer = (int64_t)cfg.world_size * cfg.max_num_batched_tokens * nmax;
    // area of the argmax exchange behind the allreduce words: [world][tokens] x 4 words (never aliased with them, so a
    // stale pair can not be taken for an arrived partial sum or the other way round)
    exchange_base_words = g->inbox_floats_per_buffer;
    for (const auto &l : L)
      if (l.op == MPK_OP_ARGMAX_EXCHANGE) {
        g->inbox_floats_per_buffer += (int64_t)cfg.world_size * cfg.max_num_batched_tokens * 4;
        // keep the second buffer on the same 4 KB alignment as the first
        g->inbox_floats_per_buffer = (g->inbox_floats_per_buffer + 1023) / 1024 * 1024;
        break;
      }

    // ---- exec layers + dependencies ------------------------------------------------
    std::vector<int> exec_of_layer(L.size(), -1);
    if (!no_batch_task()) {
      ExecLayer b;
      b.type = TASK_BATCH;
      b.reads = {ST_META_OUT};
      b.writes = {ST_META};
      g->exec.push_back(b);
    }
    for (size_t i = 0; i < L.size(); ++i) {
      if (L[i].folded) continue;
      ExecLayer e;
      e.layer = (int)i;
      std::vector<int> ins, outs;
      layer_io(L[i], &ins, &outs);
      for (int t : ins) e.reads.push_back(T[t].storage);
      for (int t : outs) e.writes.push_back(T[t].storage);
      if (!no_batch_task()) e.reads.push_back(ST_META);
      e.remote_trigger = L[i].push && !L[i].push_ll;
      exec_of_layer[i] = (int)g->exec.size();
      g->exec.push_back(e);
    }
    const int E = (int)g->exec.size();
    std::map<int, int> last_writer;
    std::map<int, std::set<int>> readers;
    std::vector<std::set<int>> deps(E);
    for (int e = 0; e < E; ++e) {
      ExecLayer &x = g->exec[e];
      for (int s : x.reads) {
        auto it = last_writer.find(s);
        if (it != last_writer.end() && it->second != e) deps[e].insert(it->second);
      }
      for (int s : x.writes) {
        auto it = last_writer.find(s);
        if (it != last_writer.end() && it->second != e) deps[e].insert(it->second);
        for (int r : readers[s]) if (r != e) deps[e].insert(r);
      }
      if (x.layer >= 0 && L[x.layer].op == MPK_OP_ALLREDUCE) deps[e].insert(exec_of_layer[L[x.layer].ar_producer]);
      for (int s : x.writes) { last_writer[s] = e; readers[s].clear(); }
      for (int s : x.reads) readers[s].insert(e);
    }
    // transitive reduction
    std::vector<std::vector<char>> anc(E, std::vector<char>(E, 0));
    for (int e = 0; e < E; ++e)
      for (int d : deps[e]) {
        anc[e][d] = 1;
        for (int k = 0; k < E; ++k) if (anc[d][k]) anc[e][k] = 1;
      }
    for (int e = 0; e < E; ++e) {
      for (int d : deps[e]) {
        bool redundant = false;
        for (int d2 : deps[e]) if (d2 != d && anc[d2][d]) redundant = true;
        if (!redundant) g->exec[e].deps.push_back(d);
      }
      if ((int)g->exec[e].deps.size() > kMaxDeps)
        return fail(MPK_ERR_UNSUPPORTED, "a layer depends on more than 3 independent producers");
    }

    // ---- tasks ---------------------------------------------------------------------
    per_worker.assign(W, {});
    per_worker_exec.assign(W, {});
    int attn_ordinal = 0;
    for (int e = 0; e < E; ++e) {
      ExecLayer &x = g->exec[e];
      rot = (e * 37) % W;
      if (x.layer < 0) {
        TaskDesc d = blank(TASK_BATCH, -1);
        put(0, d, e);
        x.type = TASK_BATCH;
        continue;
      }
      rc = emit(x.layer, e, &attn_ordinal);
      if (rc) return rc;
      if (x.num_tasks == 0) return fail(MPK_ERR_INVALID, "layer " + std::to_string(x.layer) + " produced no task");
    }
    g->attn_tickets *= std::max(attn_ordinal, 1);
    // ---- events: one per exec layer ---------------------------------------------------
    g->num_events = E;
    for (int e = 0; e < E; ++e) {
      ExecLayer &x = g->exec[e];
      for (int d : x.deps) {
        uint32_t need = (uint32_t)g->exec[d].num_tasks;
        if (g->exec[d].remote_trigger) need *= (uint32_t)cfg.world_size;
        x.dep_need.push_back(need);
      }
    }
    g->worker_begin.assign(W + 1, 0);
    for (int w = 0; w < W; ++w) {
      g->worker_begin[w] = (int32_t)g->tasks.size();
      bool observed_batch = false;   // an earlier task of this worker waited on something downstream of the batching task
      for (size_t i = 0; i < per_worker[w].size(); ++i) {
        TaskDesc d = per_worker[w][i];
        const int e = per_worker_exec[w][i];
        const ExecLayer &x = g->exec[e];
        // The attention tasks read the page tables before their own dependency wait and therefore check the
        // batching event first; once the worker has acquired any event of this iteration (every layer is
        // downstream of the batching task), that check is redundant.
        if (d.type == TASK_ATTENTION && observed_batch) d.a[A_EARLY_EV] = -1;
        if (!x.deps.empty() && x.type != TASK_BATCH && e > 0) observed_batch = true;
        for (size_t k = 0; k < x.deps.size(); ++k) {
          d.dep_event[k] = x.deps[k];
          d.dep_need[k] = x.dep_need[k];
          if (g->exec[x.deps[k]].remote_trigger) d.flags |= (TF_DEP0_REMOTE << k);
        }
        d.trig_event = e;
        if (x.remote_trigger) d.flags |= TF_REMOTE_TRIGGER;
        if (x.type == TASK_NOP) g->exec[e].type = d.type;
        g->tasks.push_back(d);
        g->task_exec.push_back(e);
      }
    }
    g->worker_begin[W] = (int32_t)g->tasks.size();
    g->general_kernel = cfg.max_num_batched_tokens > 8;
    for (const auto &d : g->tasks)
      if ((d.type == TASK_LINEAR && (d.flags & TF_FP8)) || d.type >= TASK_QUANTIZE_FP8) g->general_kernel = true;
    g->num_workers = W;
    g->world_size = std::max(cfg.world_size, 1);
    // attention ticket banks: patch the ticket offset now that the bank size is known
    const int64_t bank = attn_ordinal > 0 ? g->attn_tickets / attn_ordinal : 0;
    for (auto &d : g->tasks)
      if (d.type == TASK_ATTENTION) d.a[A_TICKET] = (int)(d.a[A_TICKET] * bank);
    return simulate_task_graph(*g, err);
  }
};

}  // namespace

void plan_silu_epilogue(const mpk_config &cfg, std::vector<TensorInfo> *tensors, std::vector<LayerInfo> *layers) {
  std::vector<TensorInfo> &T = *tensors;
  std::vector<LayerInfo> &L = *layers;
  auto uses = [&](const LayerInfo &l, int t) { for (int x : l.t) if (x == t) return true; return false; };
  for (size_t i = 0; i < L.size(); ++i) {
    LayerInfo &lin = L[i];
    if (lin.op != MPK_OP_LINEAR && lin.op != MPK_OP_RMSNORM_LINEAR) continue;
    const int wi = lin.op == MPK_OP_LINEAR ? 1 : 2, yi = lin.op == MPK_OP_LINEAR ? 2 : 3;
    if ((int)lin.t.size() <= yi || lin.t[wi] < 0 || lin.t[yi] < 0) continue;
    TensorInfo &w = T[lin.t[wi]];
    const int mid = lin.t[yi];
    if (w.owner != 3 || w.shuffle_src.size() != 2 || w.dims.size() != 2 || w.dtype != MPK_BF16 || T[mid].owner == 0) continue;
    const int64_t I = T[w.shuffle_src[0]].dim(0);
    if (T[w.shuffle_src[1]].dim(0) != I || w.dim(0) != 2 * I || I % 2 != 0) continue;
    // the weight may have no other user; the intermediate (often one buffer shared by all decoder layers) must
    // be read by exactly one silu_mul layer before anything defines it again
    auto output_of = [&](const LayerInfo &l) {
      switch (l.op) {
        case MPK_OP_LINEAR: case MPK_OP_SPLITK_LINEAR: return l.t.size() > 2 ? l.t[2] : -1;
        case MPK_OP_RMSNORM_LINEAR: case MPK_OP_LINEAR_RESIDUAL: return l.t.size() > 3 ? l.t[3] : -1;
        default: return -1;
      }
    };
    int silu = -1;
    bool ok = true;
    for (size_t j = 0; j < L.size() && ok; ++j)
      if (j != i && uses(L[j], lin.t[wi])) ok = false;
    for (size_t j = i + 1; j < L.size() && ok; ++j) {
      if (output_of(L[j]) == mid) break;                       // defined again: later readers see that value
      if (!uses(L[j], mid)) continue;
      if (L[j].op == MPK_OP_SILU_MUL && L[j].t[0] == mid && silu < 0) silu = (int)j;
      else ok = false;
    }
    if (!ok || silu < 0) continue;
    LayerInfo &s = L[silu];
    const TensorInfo &act = T[s.t[1]];
    if (std::max(s.grid[0], 1) != w.shuffle_groups || act.dims.size() != 2 || act.dim(1) != I || act.dtype != MPK_BF16) continue;
    (void)cfg;
    w.shuffle_groups = (int)(I / 2);      // 2 gate rows, then 2 up rows
    lin.silu_out = s.t[1];
    s.folded = true;
  }
}

int build_task_graph(GraphInputs in, CompiledGraph *out, std::string *err) {
  *out = CompiledGraph();
  Builder b(in, out, err);
  return b.run();
}

int simulate_task_graph(const CompiledGraph &g, std::string *err) {
  const int W = g.num_workers;
  std::vector<uint64_t> counters(g.num_events, 0);
  std::vector<int> pos(W);
  for (int w = 0; w < W; ++w) pos[w] = g.worker_begin[w];
  size_t done = 0;
  bool progress = true;
  while (progress) {
    progress = false;
    for (int w = 0; w < W; ++w) {
      while (pos[w] < g.worker_begin[w + 1]) {
        const TaskDesc &d = g.tasks[pos[w]];
        bool ready = true;
        for (int k = 0; k < kMaxDeps; ++k) {
          if (d.dep_event[k] < 0) continue;
          // a remote-triggered event also receives the peers' arrivals; count ours world times
          if (counters[d.dep_event[k]] < d.dep_need[k]) ready = false;
        }
        if (!ready) break;
        if (d.trig_event >= 0)
          // every rank runs the same graph: a remote-triggered arrival is mirrored by the peers
          counters[d.trig_event] += (d.flags & TF_REMOTE_TRIGGER) ? (uint64_t)g.world_size : 1ull;
        ++pos[w];
        ++done;
        progress = true;
      }
    }
  }
  if (done != g.tasks.size()) {
    std::ostringstream os;
    os << "task graph deadlocks in host simulation: " << done << " of " << g.tasks.size() << " tasks ran";
    for (int w = 0; w < W; ++w)
      if (pos[w] < g.worker_begin[w + 1]) {
        os << "; worker " << w << " stuck at task " << pos[w] << " (layer " << g.tasks[pos[w]].layer << ")";
        break;
      }
    *err = os.str();
    return MPK_ERR_DEADLOCK;
  }
  for (int e = 0; e < g.num_events; ++e) {
    uint64_t expect = (uint64_t)g.exec[e].num_tasks;
    if (g.exec[e].remote_trigger) expect *= (uint64_t)g.world_size;
    if (counters[e] != expect) {
      *err = "event " + std::to_string(e) + " fired " + std::to_string(counters[e]) + " times, expected " +
             std::to_string(expect);
      return MPK_ERR_DEADLOCK;
    }
  }
  return MPK_OK;
}

std::string dump_task_graph(const CompiledGraph &g, const std::vector<TensorInfo> &tensors,
                            const std::vector<LayerInfo> &layers) {
  static const char *names[] = {"nop", "batch", "embed", "rmsnorm", "linear", "attention", "silu_mul",
                                "argmax_partial", "argmax_reduce", "allreduce", "elementwise_add", "tensor_init",
                                "quantize_fp8", "moe_routing", "moe_gemm", "moe_silu_mul", "moe_mul_sum_add",
                                "mla_append", "mla_decode", "mla_reduce", "sampling_partial", "sampling_reduce", "argmax_exchange", "ar_push"};
  std::ostringstream os;
  os << "{\"num_workers\": " << g.num_workers << ", \"num_tasks\": " << g.tasks.size()
     << ", \"num_events\": " << g.num_events << ", \"num_layers\": " << layers.size()
     << ", \"num_folded\": " << g.num_folded << ", \"num_stages\": " << g.num_stages << ", \"stage_bytes\": " << g.stage_bytes
     << ", \"x_tile_bytes\": " << g.x_tile_bytes << ", \"weight_bytes\": " << g.weight_bytes
     << ",\n \"events\": [\n";
  for (size_t e = 0; e < g.exec.size(); ++e) {
    const ExecLayer &x = g.exec[e];
    os << "  {\"event\": " << e << ", \"type\": \"" << names[x.type < 24 ? x.type : 0] << "\", \"layer\": " << x.layer
       << ", \"tasks\": " << x.num_tasks << ", \"deps\": [";
    for (size_t k = 0; k < x.deps.size(); ++k) os << (k ? ", " : "") << "[" << x.deps[k] << ", " << x.dep_need[k] << "]";
    os << "]";
    if (x.layer >= 0 && layers[x.layer].prologue != PRO_PLAIN)
      os << ", \"prologue\": \"" << (layers[x.layer].prologue == PRO_RMSNORM ? "rmsnorm" : "silu_mul") << "\"";
    if (x.layer >= 0 && layers[x.layer].silu_out >= 0) os << ", \"epilogue\": \"silu_mul\"";
    if (x.remote_trigger) os << ", \"push\": true";
    if (x.tc_rows > 0) os << ", \"tcgen05\": {\"tile_rows\": " << x.tc_rows << ", \"k_blocks_per_slot\": " << x.tc_kblocks << "}";
    if (x.layer >= 0 && !layers[x.layer].t.empty()) {
      const LayerInfo &l = layers[x.layer];
      int out = l.t.back();
      if (out >= 0) os << ", \"out\": \"" << tensors[out].name << "\"";
    }
    os << "}" << (e + 1 < g.exec.size() ? ",\n" : "\n");
  }
  os << " ]}\n";
  return os.str();
}

}  // namespace mpk
