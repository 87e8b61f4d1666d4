// Tensor-parallel exchange between the ranks of one model replica (one process per GPU).
#pragma once
#include "common.cuh"

constexpr uint32_t kTpMaxWorld = 8;
constexpr uint32_t kTpMaxCtas = 64;     // CTAs of one all-reduce launch
constexpr uint32_t kTpArgmaxRows = 1024;

struct ruai_tp_state {
  uint32_t rank = 0, world = 1;
  size_t slot_floats = 0;              // floats one rank can deposit per exchange
  void* region = nullptr;              // this rank's exchange region (exported through CUDA IPC)
  size_t region_bytes = 0;
  void* peer[kTpMaxWorld] = {};        // every rank's region mapped here; peer[rank] == region
  float* partial = nullptr;            // where this rank's o_proj / down_proj partial sums land
  unsigned* seq = nullptr;             // device: [0] all-reduce sequence, [1] argmax sequence, [2..3] arrival counters
  bool connected = false;
  float* local_partial() const { return partial; }
};

int ruai_tp_init(ruai_ctx* c, ruai_tp_state* t, uint32_t rank, uint32_t world, uint32_t d);
void ruai_tp_destroy(ruai_tp_state* t);
int ruai_tp_export_handle(ruai_ctx* c, ruai_tp_state* t, void* handle_out);
int ruai_tp_connect_handles(ruai_ctx* c, ruai_tp_state* t, const void* handles);
int ruai_tp_resync_state(ruai_ctx* c, ruai_tp_state* t);
int ruai_tp_check_ready(ruai_ctx* c, ruai_tp_state* t, uint32_t rows, uint32_t d);
// x[rows, d] += sum over ranks of partial[rows, d], the same bits on every rank.
// With `sumsq` (one row, d <= 4096 only) it also leaves sum(x^2) of the new row there, as one tile.
int ruai_tp_allreduce_add(ruai_ctx* c, ruai_tp_state* t, float* x, uint32_t rows, uint32_t d, int* err, float* sumsq = nullptr);
bool ruai_tp_allreduce_gives_sumsq(uint32_t rows, uint32_t d);
// Greedy argmax over a vocabulary split by columns: out[row] = global index of the maximum.
int ruai_tp_argmax(ruai_ctx* c, ruai_tp_state* t, const float* logits, uint32_t n_local, uint32_t rows, uint32_t col_offset, int32_t* out, int* err);
