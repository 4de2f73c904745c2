// Host-side task-graph compiler: layers -> folded layers -> tasks, events, static
// per-worker schedules.
//
// Plays the role of the reference's Graph::register_task / register_mugraph /
// build_annotated_graph (src/kernel/graph.cc:439-853, src/kernel/runtime.cc:76-1017,
// src/kernel/annotated_graph.cc:101-698) without generating source code: the result is
// a flat array of TaskDesc records for one pre-built megakernel.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/mpk_b200.h"
#include "runtime_types.h"

namespace mpk {

struct TensorInfo {
  std::string name;
  void *ptr = nullptr;
  int dtype = MPK_BF16;
  std::vector<int64_t> dims, strides;
  int owner = 0;              // 0 borrowed, 1 owned, 2 owned + symmetric request, 3 owned + filled by shuffle
  std::vector<int> shuffle_src;
  int shuffle_groups = 0;
  uint64_t bytes = 0;
  int storage = -1;           // tensors sharing memory share a storage id
  int64_t dim(int i) const { return dims[i]; }
  int64_t ld() const { return dims.size() >= 2 ? strides[dims.size() - 2] : 0; }
};

// internal op: push stage of an allreduce whose input tensor was written by a layer without a push epilogue
constexpr int MPK_OP_AR_PUSH = 1000;

struct LayerInfo {
  int op = 0;
  std::vector<int> t;          // tensor ids (inputs then outputs), -1 = absent
  int grid[3] = {1, 1, 1};
  std::vector<int64_t> params;
  // set by the folding passes
  bool folded = false;         // absorbed into its consumers, emits no task
  int prologue = PRO_PLAIN;    // for linear layers
  int pro_src = -1;            // tensor the prologue reads (raw x, or gate|up buffer)
  int pro_gamma = -1;
  int pro_groups = 1;
  bool push = false;           // linear: epilogue pushes fp32 partials to the peers' inboxes
  int ar_index = -1;           // allreduce ordinal within the iteration
  int ar_producer = -1;        // allreduce: exec layer of the pushing linear
  bool push_ll = false;        // linear: push self-validating {bf16, sequence} words (allreduce fused into consumers)
  int gather_ar = -1;          // linear: its prologue gathers this allreduce's pushed partials
  int gather_res = -1;         // tensor added to the gathered sum (residual), -1: none
  int gather_out = -1;         // tensor that receives the reduced activations
  int silu_out = -1;           // linear over [gate | up] weights re-interleaved 2 + 2: its epilogue writes silu(gate) * up here
};

// One schedulable group of tasks that triggers one event.
struct ExecLayer {
  int layer = -1;              // index into layers, -1 for the batching task
  uint32_t type = TASK_NOP;
  std::vector<int> reads, writes;   // storage ids
  std::vector<int> deps;            // exec-layer indices after transitive reduction
  std::vector<uint32_t> dep_need;
  int first_task = 0, num_tasks = 0;
  bool remote_trigger = false;
  int tc_rows = 0, tc_kblocks = 0;  // tcgen05 linear: rows of a weight tile, 64-column k blocks per ring slot
};

// A 3-D tensor map over one task's weight panel, viewed as {64 columns, rows, K / 64} so that one TMA box
// {64, box_rows, box_kblocks} lands as box_kblocks swizzled [box_rows][128-byte] blocks (encoded by the C ABI layer).
struct TmapSpec {
  uint64_t base = 0;          // device address of the panel's first element
  int64_t rows = 0;           // rows of the panel (rows of a box beyond it are zero-filled, not read)
  int64_t ld_bytes = 0;       // bytes between rows
  int64_t kblocks = 0;        // K / (128 / elt_bytes)
  int box_rows = 0, box_kblocks = 0;
  int elt_bytes = 2;
};

struct CompiledGraph {
  std::vector<ExecLayer> exec;
  std::vector<TaskDesc> tasks;            // grouped by worker
  std::vector<int32_t> worker_begin;      // [W + 1]
  std::vector<int> task_exec;             // exec layer of each task (same order as tasks)
  int num_workers = 0;
  int world_size = 1;
  int num_events = 0;
  int num_folded = 0;
  int num_stages = 0;
  int stage_bytes = 0;
  int chunk_cols = 0;                     // k extent of a streamed chunk, at most
  int x_tile_bytes = 0;
  int num_allreduce = 0;
  bool general_kernel = false;            // FP8 tasks or more than 8 batched tokens: needs the general instantiation
  bool use_tmem = false;                  // some linear runs on tcgen05: workers allocate tensor memory
  int tc_tokens = 0;                      // token rows of the tcgen05 activation operand tile
  std::vector<TmapSpec> tmaps;            // indexed by TaskDesc::a[L_TMAP]
  int64_t weight_bytes = 0;
  int64_t inbox_floats_per_buffer = 0;    // world * mbt * Nmax
  int64_t attn_scratch_floats = 0;
  int64_t attn_tickets = 0;
};

struct GraphInputs {
  const mpk_config *cfg;
  const std::vector<TensorInfo> *tensors;
  std::vector<LayerInfo> *layers;
  int num_workers;
  uint64_t inbox_base_floats;   // offset of the inbox inside the exchange region, in floats
};

// Returns MPK_OK or an error; `err` receives the message.
int build_task_graph(GraphInputs in, CompiledGraph *out, std::string *err);
// Event-protocol simulation on the host (the reference runs the same kind of check at every
// compile, src/kernel/runtime.cc:962-1017): every task runs once, no worker blocks forever.
int simulate_task_graph(const CompiledGraph &g, std::string *err);
// Run before shuffled tensors are materialised: a linear whose weight is a shuffle of [gate, up] rows and whose
// output only feeds a silu_mul layer gets its weight re-interleaved as 2 gate rows + 2 up rows, so that every
// 16-row mma tile holds matching pairs and the linear's epilogue can apply the activation itself.
void plan_silu_epilogue(const mpk_config &cfg, std::vector<TensorInfo> *tensors, std::vector<LayerInfo> *layers);
std::string dump_task_graph(const CompiledGraph &g, const std::vector<TensorInfo> &tensors,
                            const std::vector<LayerInfo> &layers);

}  // namespace mpk
