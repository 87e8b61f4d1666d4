// Persistent decode step: one cooperative kernel per token instead of a chain of launches.
// Declarations shared by pstep.cu (kernel + launch), spack.cu (weight layout) and model.cu.
#pragma once
#include "common.cuh"

// "Tile stream" layout of a quantized weight, built once from the chunk layout.  The matrix is cut into
// tiles of 128 output columns; within a tile the records of consecutive blocks of k are contiguous, so
// any run of blocks of one tile is a single bulk copy:
//   int4 (group 32): record (tile, group) = 2560 bytes: 128 columns x 16 packed bytes (the chunk of that
//                    column and group, see pack.cu), then the 128 f32 scales of the group;
//   int8           : record (tile, 32 rows of k) = 4096 bytes: two halves of 16 rows, each 128 columns x
//                    16 bytes, which is the canonical K-major operand layout of tcgen05.mma as it stands.
// Columns past n hold weight 0 (and scale 0); rows past k hold 0.
struct ruai_sweight {
  uint32_t k = 0, n = 0, bits = 0;
  uint32_t ntiles = 0, nblk = 0, rec_bytes = 0;
  uint8_t* data = nullptr;          // device, [ntiles][nblk][rec_bytes]
  const float* colscale = nullptr;  // int8: f32 [n], borrowed from the chunk-layout weight
  size_t bytes = 0;
};

constexpr uint32_t kStreamTileCols = 128;
constexpr uint32_t kRingSlotBytes = 12288;  // one ring stage of the persistent kernel: 4 int4 groups (10240 B), 3 int8 blocks, or K + V rows
constexpr uint32_t kStreamRec4 = 2560, kStreamRec8 = 4096;

bool ruai_sweight_supported(const ruai_qweight* w);
int ruai_sweight_create(ruai_ctx* c, const ruai_qweight* w, ruai_sweight* out);
void ruai_sweight_free(ruai_sweight* s);

namespace ps {

constexpr int kMaxRows = 2;    // sequences per step the persistent kernel takes
constexpr int kMaxLayers = 64;  // layer pointer table kept in shared memory

// Accumulators of the split-k sums are 64-bit fixed point (value * 2^36): integer adds commute, so the
// result does not depend on the order in which CTAs (or GPUs) deliver their parts.
constexpr float kFix = 68719476736.0f;
constexpr float kUnfix = 1.0f / 68719476736.0f;

struct LayerPtrs {
  const uint8_t* w_qkv; const uint8_t* w_o; const uint8_t* w_gu; const uint8_t* w_dn;
  const float* s_qkv; const float* s_o; const float* s_gu; const float* s_dn;  // int8 column scales
  const float* n1; const float* n2;
  float* kc; float* vc;
};

struct Geom { uint32_t ntiles, nblk, n, k; };

struct StepParams {
  uint32_t m, L, d, nq, nkv, hd, Hl, KVl, rep, fl, Vl, V, cap, bits;
  uint32_t splits;          // key splits per (sequence, KV head) in the attention phase
  uint32_t keys_per_stage;  // cached keys per ring stage (K rows, then V rows)
  uint32_t col_offset;      // first vocabulary column of this rank (tensor parallel), else 0
  float eps, attn_scale;
  Geom qkv, o, gu, dn, head;
  const LayerPtrs* layers;  // device, [L]
  const uint8_t* w_head; const float* s_head;
  const float* final_norm; const float* embed; const float2* rope;
  int32_t* ids; int32_t* len; int* err;
  float* x0; float* x1;
  float* ss_a; float* ss_b; float* ss_c;  // per-group sums of squares [m][d/32] written by the norm loaders
  long long* acc_qkv; long long* acc_o; long long* acc_gu; long long* acc_dn; long long* acc_logits;
  int* poison;              // [5][kMaxRows]: non-finite partial sums seen for an accumulator row
  float* att_part;          // attention partials [m*KVl*splits][rep][hd + 4]
  float* att_out;           // merged attention output [m][nq], f32
  unsigned* att_cnt;        // [m*KVl] splits that have finished an item; back to zero when the item is merged
  float* logits;            // f32 [m][Vl]
  int2* arg_slots;          // [gridDim][kMaxRows] best (ordered value, column) per CTA
  unsigned* bar;            // grid barrier counter (monotonic)
  unsigned bar_base;        // its value when this launch starts
  int* status;              // context status word: 3 = a bounded wait ran out
  int* abort_flag;          // set by the first CTA that gives up; everyone else leaves at its next wait
  unsigned spin_limit;      // polls of a grid-barrier wait
  unsigned tx_shortfall;    // failure injection (host-made): the first stage's copy is announced this many bytes too large
  int want_argmax;
  unsigned long long* trace;  // profiling builds (RUAI_B200_TRACE): per-stage clock stamps of CTA 0, else unused
};

// One generic quantized GEMV as its own (test / microbenchmark) program: out[m][n] = x[m][k] @ W.
struct GemvTestParams {
  uint32_t m, repeat;
  Geom g; uint32_t bits;
  const uint8_t* w; const float* colscale;
  const float* x;        // f32 [m][k]
  long long* acc;        // [m][n], zero on entry; left zero on exit
  int* poison;           // [kMaxRows]
  float* out;            // f32 [m][n]
  unsigned* bar; unsigned bar_base; int* status; int* abort_flag; unsigned spin_limit;
  unsigned tx_shortfall;
  unsigned long long* trace;
};

}  // namespace ps

struct ruai_pstep_buffers;  // device buffers of one model's persistent step (pstep.cu)

int ruai_pstep_launch(ruai_ctx* c, const ps::StepParams& p);
int ruai_pgemv_launch(ruai_ctx* c, const ps::GemvTestParams& p);
// CTAs of the persistent kernels on this device (one per SM), 0 if the kernel cannot be resident.
int ruai_pstep_grid(ruai_ctx* c);
