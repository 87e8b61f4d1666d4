// The persistent decode step: ONE cooperative kernel per generated token.
//
// It runs, for Llama-shaped models and up to two sequences, what Llama::run (src/nn/modules/llama.rs:441-463;
// DecoderLayer::forward 306-309; Attention::forward 248-277) does per token: per layer q/k/v Linear, RoPE + KV append +
// attention, o_proj, gate/up Linear + SwiGLU, down_proj, then the head and the greedy pick (generation.rs:6-8).  One CTA
// per SM stays resident for the whole step and walks these as PHASES separated by a grid-wide barrier.  It is the
// alternative to the chain of launches of model.cu (one kernel per Linear / attention); which of the two a model uses is
// the caller's choice (ruai_model_use_persistent_step), the chain being the default because it is the faster one on the
// shapes measured so far: a phase boundary here (last partial sums out -> grid barrier -> activations back from L2 ->
// digits -> first MMAs) costs about as much as a launch boundary there, and the chain's GEMV kernels keep more expanding
// warps per SM busy.
//
// The weights never stop streaming.  Every CTA owns, per phase, a contiguous run of (128-column tile, block of k) units
// of the weight in the tile-stream layout (pstep.cuh).  One producer thread walks the stages of the WHOLE step and keeps
// a ring of 12 KB bulk copies (cp.async.bulk + mbarrier) full; it is held back only by free ring slots, never by a phase
// boundary, so while the CTAs meet at a barrier the next phase's weights (or the next layer's cached keys and values)
// are already landing in shared memory.  With each stage it leaves a small record (tile, window slot, blocks), from
// which the other roles take what the stage holds: nobody but the producer walks the stage list.
//
// Arithmetic of a GEMV phase is that of gemv_tc.cu / gemv_tc8.cu: activations as block fixed point (int4: three int8
// digits per group of 32; int8: four digits per row of the CTA's window), exact integer products on the tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), one f32 multiply-add per (scale group, column, row).  The warps
// of a CTA meet only at mbarriers:
//   warp 0, one thread        : producer;
//   warps 1 and 2, one thread : MMA issuers (stage s is issued by issuer s % 2; a thread needs well over a hundred
//                               cycles per tcgen05.mma);
//   warps 3..14               : three warpgroups; stage s belongs to warpgroup s % 3, which expands its int4 nibbles to
//                               bytes (one of two A-operand buffers per warpgroup) and later reads its sums out of tensor
//                               memory, scales and accumulates them (int8 needs no expansion: the ring slot IS the
//                               operand, and warpgroups 0 / 1 read out issuer 0's / 1's runs);
//   warps 1..14 together      : the digits of the activations at the start of a phase, the attention phase, the logits.
// A CTA's partial sums of a tile go to a 64-bit fixed-point accumulator in global memory with red.add.u64: integer
// addition commutes, so the result is bit-identical from run to run whatever the arrival order.  Everything non-linear
// happens when the NEXT phase loads its activations ("loaders"): residual add, RMSNorm weight (the 1/rms factor is a
// per-row scalar and is applied one phase later, from per-group sums of squares the loader leaves), SwiGLU.  The
// attention phase works one (sequence, KV head, key split) item per CTA; the split that finishes an item last merges it.
//
// Two things the kernel is built around, both measured: (1) no stack.  Nearly all of the SM's memory is configured as
// shared memory, the L1 that is left holds no per-thread stack, and every touch of a spilled register or a by-reference
// struct costs a trip to L2 (a few hundred bytes of stack frame doubled the step time).  Hence the phase descriptor and
// the common parameters in shared memory, streaming state scoped after the conversion, small batches where registers
// run out.  (2) No test in front of loads where a stage is full: the copy of a loop without the per-group condition
// lets the compiler issue the loads together.
//
// Every wait is bounded (mbarrier waits, the grid barrier); a wait that runs out sets an abort flag that the other CTAs
// see at their next wait, the kernel frees its tensor memory and returns, and the host reports RUAI_ERR_TIMEOUT.
#include <algorithm>
#include <type_traits>

#include "pipeline.cuh"
#include "pstep.cuh"

namespace ps {

using namespace pipe;

constexpr int kCols = 128;            // tile columns = MMA M = TMEM lanes
constexpr int kStage4 = 4;            // int4 scale groups per ring stage: the unit one warpgroup works on
constexpr int kStage8 = 3;            // int8 32-row blocks per ring stage
constexpr uint32_t kSlotBytes = kRingSlotBytes;
constexpr int kSlots = 7;
constexpr int kGroups = 3;            // warpgroups of four warps; ring stage s belongs to warpgroup s % kGroups
constexpr uint32_t kABufBytes = kStage4 * 4096;  // A-operand buffer of one stage; two per warpgroup
constexpr uint32_t kAcc8 = 8;         // int8: independent accumulators a warpgroup's MMAs rotate through
constexpr int kWin = 128;             // window of the activation digits: groups (int4) / blocks (int8)
constexpr uint32_t kBRec = 256;       // digit operand of one group: [2 k-halves][8 rows][16 bytes]
// 15 warps: at most four on an SM sub-partition, so its 16 K registers allow 128 per thread (a sixteenth warp fits; a
// seventeenth would cut every thread to 96 registers, and the spills that follow cost more than the warps bring).
constexpr int kThreads = 480;         // warp 0: producer; warp 1: leader + MMA issuer 0; warp 2: MMA issuer 1; warps 3..14: three warpgroups
constexpr int kConsumers = 448;       // warps 1..14
constexpr int kConvWarps = 14;
constexpr int kWarpLeader = 1, kWarpIssuer1 = 2, kWarpWg0 = 3;
constexpr int kLeaderTid = kWarpLeader * 32;
constexpr uint32_t kTmemCols = 512;

constexpr size_t kOffSlots = 0;
constexpr size_t kOffABuf = kOffSlots + (size_t)kSlots * kSlotBytes;
constexpr size_t kOffBWin = kOffABuf + 2 * (size_t)kGroups * kABufBytes;
constexpr size_t kOffMeta = kOffBWin + (size_t)kWin * kBRec;
constexpr size_t kOffLayers = kOffMeta + (size_t)kWin * kMaxRows * 8;

enum { PH_GEMV = 0, PH_ATTN = 1, PH_FINAL = 2, PH_PICK = 3, PH_OUT = 4 };
enum { LD_PLAIN = 0, LD_EMBED = 1, LD_RESID = 2, LD_SWIGLU = 3 };

struct PhaseDesc {
  int type;
  // GEMV
  const uint8_t* w; const float* colscale;
  uint32_t ntiles, nblk, n, k, bits;
  int loader;
  const float* norm_w;        // RMSNorm weight multiplied into the digits (NULL: none)
  const float* x_in; float* x_out;
  const long long* acc_in; const int* poison_in; uint32_t in_ld;
  float* ss_out;              // [m][k/32] sums of squares of the x this loader builds
  const float* ss_in; uint32_t ss_groups; float ss_dim;  // source of this phase's 1/rms factor
  long long* acc_out; int* poison_out;
  long long* zero0; uint32_t zero0_n; int* zero0_poison;
  long long* zero1; uint32_t zero1_n; int* zero1_poison;
  // ATTN
  float* kc; float* vc;
};

// What the kernel needs from its parameter block whichever program it runs.
struct Common {
  uint32_t m;
  unsigned* bar; unsigned bar_base; int* status; int* abort_flag; unsigned spin_limit;
  unsigned tx_shortfall;  // failure injection: see StepParams
  // attention / final (step program only)
  const StepParams* sp;
  float* out;  // test program: f32 [m][n]
  unsigned long long* trace;
};

struct Bars {
  uint64_t full[kSlots], empty[kSlots];
  uint64_t a_ready[kGroups][2];   // a warpgroup's A buffer 0 / 1 is written (its 4 warps arrive); one barrier per buffer,
                                  // because a warpgroup may be a stage ahead of the issuer
  uint64_t mma_done[kGroups][2];  // the MMAs of a warpgroup's stage into accumulator buffer 0 / 1 have completed
  uint64_t seg_done[2][2];        // int8: the MMAs of an issuer's part of a run (into accumulator set 0 / 1) have completed
  uint64_t seg_free[2][2];        // int8: the sums of that set are read out (the 4 warps of warpgroup 0 / 1 arrive)
  uint64_t fin[2];                // every MMA of an issuer has completed (before the tensor memory goes back)
};

// The phase descriptors and the common parameters live in shared memory: with nearly all of the SM's memory configured
// as shared memory the L1 is small, per-thread stack slots fall out of it, and each later touch of one costs a trip to L2.
struct Shared {
  Bars b;
  PhaseDesc D[3];             // the consumers' phase p descriptor is D[p % 3], written during phase p - 1 by a spare lane
  PhaseDesc Dp;               // the producer's (it runs ahead)
  Common c;
  uint2 rec[kSlots];          // per ring slot, left by the producer: x = tile, y = window slot | blocks << 16
  uint32_t wgrec[kGroups][2]; // per A buffer, left by the warpgroup for the issuer: window slot | blocks << 16
  uint4 segrec[2][2];         // int8, per issuer and accumulator set: x = tile, y = MMAs of the run, z = last run of the round
  uint32_t tmem;
  volatile int abort;
  int att_last;                // attention: this CTA completed its item and merges the splits
  float wmax[kMaxRows][kConvWarps];
  float xscale[kMaxRows];
  int2 arg[kMaxRows][kConvWarps];
};

// ---- small device helpers --------------------------------------------------------------------

// Named barrier over `count` threads (whole warps).  bar.sync is warp-aligned, so lanes that took a single-lane
// branch just before meet the rest of their warp first.
__device__ __forceinline__ void bar_sync(int id, int count) {
  __syncwarp();
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void red_add_s64(long long* p, long long v) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_inc(unsigned* p) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ float unfix(long long v) { return __ll2float_rn(v) * kUnfix; }
__device__ __forceinline__ float silu_ref(float v) { return v * (1.0f / (1.0f + expf(-v))); }  // ops.rs:158-160
__device__ __forceinline__ int32_t ordered_bits(float v) {  // f32::total_cmp order as a signed integer
  int32_t i = __float_as_int(v);
  return i ^ (int32_t)(((uint32_t)(i >> 31)) >> 1);
}
__device__ __forceinline__ bool finite_f(float v) { return fabsf(v) <= 3.402823466e38f; }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}

// ---- the units of one CTA in one GEMV phase ---------------------------------------------------

// Units are (tile, block) in tile-major order; CTA b owns units [U*b/G, U*(b+1)/G).  Digits of the
// activations are kept for a window of kWin blocks: if the weight has at most kWin blocks of k the window
// slot of a block is the block itself and the phase is one round; otherwise a round is kWin consecutive units.
struct StageIter {
  uint32_t u0, u1, blk_at_u0;
  bool windowed;
  __device__ void init(uint32_t ntiles, uint32_t nblk) {
    const uint64_t units = (uint64_t)ntiles * nblk;
    u0 = (uint32_t)(units * blockIdx.x / gridDim.x);
    u1 = (uint32_t)(units * (blockIdx.x + 1) / gridDim.x);
    blk_at_u0 = u0 % nblk;
    windowed = nblk > (uint32_t)kWin;
  }
};

// ---- key/value stages of the attention phase ----------------------------------------------------

struct AttnPlan {
  uint32_t n_items, S, KS, n_cached, per;
  __device__ void init(uint32_t m, uint32_t KVl, uint32_t splits, uint32_t keys_per_stage, uint32_t len) {
    S = splits; KS = keys_per_stage; n_items = m * KVl * splits; n_cached = len;
    per = (len + splits - 1) / splits;
  }
  __device__ void range(uint32_t item, uint32_t& k0, uint32_t& k1) const {
    const uint32_t split = item % S;
    k0 = min(n_cached, split * per);
    k1 = min(n_cached, k0 + per);
  }
  __device__ uint32_t stages(uint32_t item) const {
    uint32_t k0, k1;
    range(item, k0, k1);
    return (k1 - k0 + KS - 1) / KS;
  }
};

// ---- programs -------------------------------------------------------------------------------------

struct StepProgram {
  const StepParams& P;
  const LayerPtrs* lay;  // shared-memory copy
  __device__ uint32_t nphases() const { return 5u * P.L + 3u; }
  __device__ void get(uint32_t p, PhaseDesc& D) const {
    D = PhaseDesc();
    const uint32_t MT = kMaxRows;
    D.zero0 = nullptr; D.zero1 = nullptr; D.zero0_n = 0; D.zero1_n = 0;
    if (p < 5u * P.L) {
      const uint32_t l = p / 5u, kind = p - 5u * l;
      const LayerPtrs& Y = lay[l];
      D.bits = P.bits;
      switch (kind) {
        case 0:  // q/k/v Linear on RMSNorm(x); x = embedding (layer 0) or x + down_proj of the previous layer
          D.type = PH_GEMV; D.w = Y.w_qkv; D.colscale = Y.s_qkv;
          D.ntiles = P.qkv.ntiles; D.nblk = P.qkv.nblk; D.n = P.qkv.n; D.k = P.qkv.k;
          D.loader = l == 0 ? LD_EMBED : LD_RESID; D.norm_w = Y.n1; D.x_in = P.x0; D.x_out = P.x1;
          D.acc_in = P.acc_dn; D.poison_in = P.poison + 3 * MT; D.in_ld = P.d; D.ss_out = P.ss_a;
          D.acc_out = P.acc_qkv; D.poison_out = P.poison + 0 * MT;
          D.zero0 = P.acc_o; D.zero0_n = P.m * P.d; D.zero0_poison = P.poison + 1 * MT;
          break;
        case 1:  // RoPE, KV append, attention over the cache
          D.type = PH_ATTN; D.kc = Y.kc; D.vc = Y.vc;
          D.acc_in = P.acc_qkv; D.poison_in = P.poison + 0 * MT; D.in_ld = P.qkv.n;
          D.ss_in = P.ss_a; D.ss_groups = P.d / 32; D.ss_dim = (float)P.d;
          D.zero0 = P.acc_gu; D.zero0_n = P.m * P.gu.n; D.zero0_poison = P.poison + 2 * MT;
          if (l == 0) { D.zero1 = P.acc_logits; D.zero1_n = P.m * P.Vl; D.zero1_poison = P.poison + 4 * MT; }
          break;
        case 2:  // o_proj on the merged attention output
          D.type = PH_GEMV; D.w = Y.w_o; D.colscale = Y.s_o;
          D.ntiles = P.o.ntiles; D.nblk = P.o.nblk; D.n = P.o.n; D.k = P.o.k;
          D.loader = LD_PLAIN; D.x_in = P.att_out; D.in_ld = P.nq;
          D.acc_out = P.acc_o; D.poison_out = P.poison + 1 * MT;
          D.zero0 = P.acc_dn; D.zero0_n = P.m * P.d; D.zero0_poison = P.poison + 3 * MT;
          break;
        case 3:  // gate/up Linear on RMSNorm(x + o_proj)
          D.type = PH_GEMV; D.w = Y.w_gu; D.colscale = Y.s_gu;
          D.ntiles = P.gu.ntiles; D.nblk = P.gu.nblk; D.n = P.gu.n; D.k = P.gu.k;
          D.loader = LD_RESID; D.norm_w = Y.n2; D.x_in = P.x1; D.x_out = P.x0;
          D.acc_in = P.acc_o; D.poison_in = P.poison + 1 * MT; D.in_ld = P.d; D.ss_out = P.ss_b;
          D.acc_out = P.acc_gu; D.poison_out = P.poison + 2 * MT;
          D.zero0 = P.acc_qkv; D.zero0_n = P.m * P.qkv.n; D.zero0_poison = P.poison + 0 * MT;
          break;
        default:  // down_proj on silu(gate) * up
          D.type = PH_GEMV; D.w = Y.w_dn; D.colscale = Y.s_dn;
          D.ntiles = P.dn.ntiles; D.nblk = P.dn.nblk; D.n = P.dn.n; D.k = P.dn.k;
          D.loader = LD_SWIGLU; D.acc_in = P.acc_gu; D.poison_in = P.poison + 2 * MT; D.in_ld = P.gu.n;
          D.ss_in = P.ss_b; D.ss_groups = P.d / 32; D.ss_dim = (float)P.d;
          D.acc_out = P.acc_dn; D.poison_out = P.poison + 3 * MT;
          break;
      }
      return;
    }
    const uint32_t t = p - 5u * P.L;
    if (t == 0) {  // the head (int8 even for an int4 model, llama.rs:535-542) on RMSNorm(x + down_proj)
      D.type = PH_GEMV; D.bits = 8; D.w = P.w_head; D.colscale = P.s_head;
      D.ntiles = P.head.ntiles; D.nblk = P.head.nblk; D.n = P.head.n; D.k = P.head.k;
      D.loader = LD_RESID; D.norm_w = P.final_norm; D.x_in = P.x0; D.x_out = nullptr;
      D.acc_in = P.acc_dn; D.poison_in = P.poison + 3 * MT; D.in_ld = P.d; D.ss_out = P.ss_c;
      D.acc_out = P.acc_logits; D.poison_out = P.poison + 4 * MT;
    } else if (t == 1) {
      D.type = PH_FINAL;
      D.acc_in = P.acc_logits; D.poison_in = P.poison + 4 * MT; D.in_ld = P.Vl;
      D.ss_in = P.ss_c; D.ss_groups = P.d / 32; D.ss_dim = (float)P.d;
      D.zero0 = P.acc_dn; D.zero0_n = P.m * P.d; D.zero0_poison = P.poison + 3 * MT;
    } else {
      D.type = PH_PICK;
    }
  }
};

struct TestProgram {
  const GemvTestParams& P;
  __device__ uint32_t nphases() const { return 2u * P.repeat; }
  __device__ void get(uint32_t p, PhaseDesc& D) const {
    D = PhaseDesc();
    D.zero0 = nullptr; D.zero1 = nullptr; D.zero0_n = 0; D.zero1_n = 0;
    D.bits = P.bits;
    if ((p & 1u) == 0) {
      D.type = PH_GEMV; D.w = P.w; D.colscale = P.colscale;
      D.ntiles = P.g.ntiles; D.nblk = P.g.nblk; D.n = P.g.n; D.k = P.g.k;
      D.loader = LD_PLAIN; D.x_in = P.x; D.in_ld = P.g.k;
      D.acc_out = P.acc; D.poison_out = P.poison;
    } else {
      D.type = PH_OUT; D.acc_in = P.acc; D.poison_in = P.poison; D.n = P.g.n;
    }
  }
};

// Profiling builds only (-DRUAI_B200_TRACE): CTA 0 stamps its SM clock at the hand-overs of the first stages.
// Layout: stage events [kTraceStages][8], then phase events [kTracePhases][4].
#ifdef RUAI_B200_TRACE
constexpr uint32_t kTraceStages = 192, kTracePhases = 192;
#define PS_TRACE_STAGE(X, stage, ev)                                                                       \
  do {                                                                                                     \
    if ((X).c.trace && blockIdx.x == 0 && (stage) < kTraceStages) (X).c.trace[(size_t)(stage) * 8 + (ev)] = clock64(); \
  } while (0)
#define PS_TRACE_PHASE(X, phase, ev)                                                                       \
  do {                                                                                                     \
    if ((X).c.trace && blockIdx.x == 0 && (phase) < kTracePhases) (X).c.trace[(size_t)kTraceStages * 8 + (size_t)(phase) * 4 + (ev)] = clock64(); \
  } while (0)
#define PS_TRACE_ISSUE(X, stage, ev)                                                                       \
  do {                                                                                                     \
    if ((X).c.trace && blockIdx.x == 0 && (stage) < kTraceStages)                                          \
      (X).c.trace[(size_t)kTraceStages * 8 + (size_t)kTracePhases * 4 + (size_t)(stage) * 8 + (ev)] = clock64(); \
  } while (0)
#else
#define PS_TRACE_ISSUE(X, stage, ev) do { } while (0)
#define PS_TRACE_STAGE(X, stage, ev) do { } while (0)
#define PS_TRACE_PHASE(X, phase, ev) do { } while (0)
#endif

// ---- the kernel body ------------------------------------------------------------------------------

template <int MT>
struct Ctx {
  unsigned char* smem;
  Shared* sh;
  const Common& c;
  int tid, lane, warp;
  uint32_t cur_phase;
  uint32_t s;    // ring stages so far (all kinds, all warpgroups)
  uint32_t mc0, mc1, mc2;  // int4 stages of warpgroup 0 / 1 / 2 so far (every consumer thread keeps all three)
  uint32_t sgc;  // int8 runs closed so far (issuer i and warpgroup i count the same runs)
  uint32_t tmem;
  __device__ Ctx(unsigned char* smem_, Shared* sh_) : smem(smem_), sh(sh_), c(sh_->c) {}

  __device__ unsigned char* slot_ptr(uint32_t stage) const { return smem + kOffSlots + (size_t)(stage % kSlots) * kSlotBytes; }
  __device__ unsigned char* abuf_ptr(uint32_t wg, uint32_t k) const { return smem + kOffABuf + (size_t)(2u * wg + (k & 1u)) * kABufBytes; }
  __device__ unsigned char* bwin() const { return smem + kOffBWin; }
  __device__ float* mscale() const { return reinterpret_cast<float*>(smem + kOffMeta); }
  __device__ int* msum() const { return reinterpret_cast<int*>(smem + kOffMeta) + kWin * kMaxRows; }
  __device__ bool aborted() const { return sh->abort != 0; }
  __device__ void give_up(int code) {
    sh->abort = 1;
    atomicExch(c.abort_flag, 1);
    atomicCAS(c.status, 0, code);
  }
  // Bounded mbarrier wait that also ends when the CTA has given up; after a failure every later wait falls
  // through, so that all warps run to the end of the program and the CTA can leave.
  __device__ bool wait(uint64_t* bar, uint32_t parity, int code) {
    if (aborted()) return false;
    const uint32_t a = smem_u32(bar);
    uint32_t ok;
    // the common case is "already complete": a plain test returns at once
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
    // otherwise poll with a short sleep in between: a suspending try_wait was seen to wake up more than a thousand cycles
    // after the barrier completed, and a tight polling loop takes the issue slots of the warps it waits for
    for (unsigned i = 0; i < c.spin_limit; ++i) {
      __nanosleep(40);
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(a), "r"(parity)
          : "memory");
      if (ok) return true;
      if ((i & 7u) == 7u && aborted()) return false;
    }
    give_up(code);
    return false;
  }
};

// Grid-wide barrier: the p-th one of this launch is passed when the counter reaches base + p * gridDim.
template <int MT>
__device__ void grid_barrier(Ctx<MT>& X, uint32_t p, bool wait_for_it) {
  __threadfence();
  red_release_gpu_inc(X.c.bar);
  if (!wait_for_it || X.aborted()) return;
  const unsigned target = X.c.bar_base + p * gridDim.x;
  for (unsigned i = 0; i < X.c.spin_limit; ++i) {
    if ((int)(ld_acquire_gpu(X.c.bar) - target) >= 0) return;
    if ((i & 63u) == 63u && __ldcg(X.c.abort_flag)) { X.sh->abort = 1; return; }
    __nanosleep(20);
  }
  X.give_up(4);
}

// ---- loaders: the activations of one group of 32 as the consuming phase needs them -----------------

// The phase's 1/rms factors (functional.rs:151-165: 1 / sqrt(mean(x^2) + eps)) from the per-group sums of squares, in
// a fixed order.  Every warp works them out for itself (same loads, same order, same result): no shared memory, no
// barrier, and the loads overlap with whatever the warp has in flight.
template <int MT>
__device__ __forceinline__ void warp_rstd(const Ctx<MT>& X, const PhaseDesc& D, float (&rs)[MT]) {
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    float s = 0.0f;
    if ((uint32_t)r < X.c.m)
      for (uint32_t i = X.lane; i < D.ss_groups; i += 32) s += __ldcg(D.ss_in + (size_t)r * D.ss_groups + i);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
    rs[r] = 1.0f / sqrtf(s * (1.0f / D.ss_dim) + X.c.sp->eps);
  }
}

// This lane's four values (k = 32 g + 4 l8 ...) of every row, as the digits are taken from them (before the RMSNorm weight).
template <int MT>
__device__ __forceinline__ void load_group(const Ctx<MT>& X, const PhaseDesc& D, uint32_t g, uint32_t l8, const float (&rs)[MT], const bool (&poisoned)[MT],
                                           float4 (&v)[MT]) {
  const uint32_t m = X.c.m;
  const uint32_t kidx = g * 32u + 4u * l8;
  const StepParams* P = X.c.sp;
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((uint32_t)r < m && kidx < D.k) {
      switch (D.loader) {
        case LD_PLAIN:
          o = __ldcg(reinterpret_cast<const float4*>(D.x_in + (size_t)r * D.in_ld + kidx));
          break;
        case LD_EMBED: {  // Embedding::forward (layers.rs:436-446)
          int32_t id = P->ids[r];
          if (id < 0 || (uint32_t)id >= P->V) { if (l8 == 0) atomicExch(P->err, 1); id = 0; }
          o = __ldg(reinterpret_cast<const float4*>(P->embed + (size_t)id * D.in_ld + kidx));
          break;
        }
        case LD_RESID: {  // x + the finished sums of the previous Linear (llama.rs:306-309)
          const float4 xv = __ldcg(reinterpret_cast<const float4*>(D.x_in + (size_t)r * D.in_ld + kidx));
          const longlong2* a = reinterpret_cast<const longlong2*>(D.acc_in + (size_t)r * D.in_ld + kidx);
          const longlong2 a0 = __ldcg(a), a1 = __ldcg(a + 1);
          o = make_float4(xv.x + unfix(a0.x), xv.y + unfix(a0.y), xv.z + unfix(a1.x), xv.w + unfix(a1.y));
          if (poisoned[r]) o.x = __int_as_float(0x7fc00000);
          break;
        }
        default: {  // LD_SWIGLU: silu(gate) * up (layers.rs:573-576); columns (2i, 2i+1) = (gate_i, up_i)
          const longlong2* a = reinterpret_cast<const longlong2*>(D.acc_in + (size_t)r * D.in_ld + 2u * kidx);
          const longlong2 a0 = __ldcg(a), a1 = __ldcg(a + 1), a2 = __ldcg(a + 2), a3 = __ldcg(a + 3);
          o.x = silu_ref(unfix(a0.x) * rs[r]) * (unfix(a0.y) * rs[r]);
          o.y = silu_ref(unfix(a1.x) * rs[r]) * (unfix(a1.y) * rs[r]);
          o.z = silu_ref(unfix(a2.x) * rs[r]) * (unfix(a2.y) * rs[r]);
          o.w = silu_ref(unfix(a3.x) * rs[r]) * (unfix(a3.y) * rs[r]);
          if (poisoned[r]) o.x = __int_as_float(0x7fc00000);
          break;
        }
      }
    }
    v[r] = o;
  }
}

// int4: block fixed point per group of 32 (gemv_tc.cu): x = f * 2^(e-20), f as three balanced base-128 digits.
template <int MT>
__device__ __forceinline__ void digits4(const Ctx<MT>& X, const float4 (&xv)[MT], uint32_t ws, int lane, bool valid) {
  const uint32_t l8 = lane & 7u;
  unsigned char* bg = X.bwin() + (size_t)ws * kBRec + (l8 >> 2) * 128u + ((4u * l8) & 15u);
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    const float vv[4] = {xv[r].x, xv[r].y, xv[r].z, xv[r].w};
    float gmax = fmaxf(fmaxf(fabsf(vv[0]), fabsf(vv[1])), fmaxf(fabsf(vv[2]), fabsf(vv[3])));
    bool bad = !(finite_f(vv[0]) && finite_f(vv[1]) && finite_f(vv[2]) && finite_f(vv[3]));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 1));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 2));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 4));
    const unsigned badmask = __ballot_sync(0xFFFFFFFFu, bad);
    bad = ((badmask >> (lane & 24)) & 0xFFu) != 0u;
    const uint32_t eb = __float_as_uint(gmax) >> 23;
    const bool nz = eb >= 20u && eb < 255u && !bad;
    const float up = nz ? __uint_as_float((273u - eb) << 23) : 0.0f;
    float xscale = nz ? __uint_as_float((eb - 19u) << 23) : 0.0f;
    if (bad) xscale = __int_as_float(0x7fc00000);  // NaN / Inf in the group: the row's sums become NaN, as in f32 arithmetic
    uint32_t w0 = 0, w1 = 0, w2 = 0;
    int fs = 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int f = __float2int_rn(vv[t] * up);
      const int d2 = ((f + 64) & 127) - 64;
      const int t1 = (f - d2) >> 7;
      const int d1 = ((t1 + 64) & 127) - 64;
      const int d0 = (t1 - d1) >> 7;
      fs += f;
      w0 |= (uint32_t)(d0 & 0xFF) << (8 * t);
      w1 |= (uint32_t)(d1 & 0xFF) << (8 * t);
      w2 |= (uint32_t)(d2 & 0xFF) << (8 * t);
    }
    fs += __shfl_xor_sync(0xFFFFFFFFu, fs, 1);
    fs += __shfl_xor_sync(0xFFFFFFFFu, fs, 2);
    fs += __shfl_xor_sync(0xFFFFFFFFu, fs, 4);
    if (valid) {
      *reinterpret_cast<uint32_t*>(bg + (3 * r + 0) * 16) = w0;
      *reinterpret_cast<uint32_t*>(bg + (3 * r + 1) * 16) = w1;
      *reinterpret_cast<uint32_t*>(bg + (3 * r + 2) * 16) = w2;
      if (l8 == 0) {
        X.mscale()[ws * MT + r] = xscale;
        X.msum()[ws * MT + r] = fs;
      }
    }
  }
}

// int8: one exponent per row for the whole window (gemv_tc8.cu): x = f * 2^(e-27), four digits.
template <int MT>
__device__ __forceinline__ void digits8(const Ctx<MT>& X, const float4 (&xv)[MT], const float (&up)[MT], uint32_t ws, int lane) {
  const uint32_t l8 = lane & 7u;
  unsigned char* bg = X.bwin() + (size_t)ws * kBRec + (l8 >> 2) * 128u + ((4u * l8) & 15u);
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    int f[4] = {__float2int_rn(xv[r].x * up[r]), __float2int_rn(xv[r].y * up[r]), __float2int_rn(xv[r].z * up[r]), __float2int_rn(xv[r].w * up[r])};
#pragma unroll
    for (int t = 3; t >= 0; --t) {  // least significant digit first; operand rows: most significant first
      uint32_t pack = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int dgt = t > 0 ? ((f[e] + 64) & 127) - 64 : f[e];
        f[e] = (f[e] - dgt) >> 7;
        pack |= (uint32_t)(dgt & 255) << (8 * e);
      }
      *reinterpret_cast<uint32_t*>(bg + (4 * r + t) * 16) = pack;
    }
  }
}

// One pass of a converter warp: four groups (8 lanes each) loaded as the phase's loader says; the loader that builds x
// also writes it back and leaves the group's sum of squares, for the groups whose (tile 0, group) unit belongs to this
// CTA (exactly one CTA per group); then the RMSNorm weight.  Returns the window slot of the lane's group.
template <int MT>
__device__ __forceinline__ uint32_t load_pass(const Ctx<MT>& X, const PhaseDesc& D, const StageIter& it, uint32_t blk0, uint32_t cnt, uint32_t i,
                                              const float (&rs)[MT], const bool (&poisoned)[MT], float4 (&xv)[MT], bool& valid) {
  const int lane = X.lane;
  const uint32_t l8 = lane & 7u, m = X.c.m;
  valid = i < cnt;
  uint32_t g = blk0 + i;
  if (g >= D.nblk) g -= D.nblk;
  const uint32_t ws = it.windowed ? i : g;
  if (!valid) {
#pragma unroll
    for (int r = 0; r < MT; ++r) xv[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    return ws;
  }
  // the weight's load goes out with the others, not after them
  float4 nw = make_float4(1.f, 1.f, 1.f, 1.f);
  if (D.norm_w) nw = __ldg(reinterpret_cast<const float4*>(D.norm_w + g * 32u + 4u * l8));
  load_group<MT>(X, D, g, l8, rs, poisoned, xv);
  if (D.ss_out) {
    const bool owner = g >= it.u0 && g < it.u1;
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      const float4 o = xv[r];
      float q = fmaf(o.x, o.x, fmaf(o.y, o.y, fmaf(o.z, o.z, o.w * o.w)));
      q += __shfl_xor_sync(0xFFu << (lane & 24), q, 1);
      q += __shfl_xor_sync(0xFFu << (lane & 24), q, 2);
      q += __shfl_xor_sync(0xFFu << (lane & 24), q, 4);
      if (owner && (uint32_t)r < m) {
        if (D.x_out) *reinterpret_cast<float4*>(D.x_out + (size_t)r * D.in_ld + g * 32u + 4u * l8) = o;
        if (l8 == 0) D.ss_out[(size_t)r * (D.k / 32u) + g] = q;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < MT; ++r) { xv[r].x *= nw.x; xv[r].y *= nw.y; xv[r].z *= nw.z; xv[r].w *= nw.w; }
  return ws;
}

// Writes the digits of one round (all consumer warps call it).
template <int MT>
__device__ __forceinline__ void convert_round(Ctx<MT>& X, const PhaseDesc& D, const StageIter& it, uint32_t blk0, uint32_t cnt) {
  const int cw = X.warp - kWarpLeader, lane = X.lane;
  const uint32_t sgi = lane >> 3;
  constexpr int kPasses = (kWin + 4 * kConvWarps - 1) / (4 * kConvWarps);  // every consumer warp converts 4 groups per pass
  float rs[MT];
  bool poisoned[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) { rs[r] = 0.0f; poisoned[r] = false; }
  if (D.poison_in) {
#pragma unroll
    for (int r = 0; r < MT; ++r) poisoned[r] = (uint32_t)r < X.c.m && __ldcg(D.poison_in + r) != 0;
  }
  if (D.ss_in) warp_rstd<MT>(X, D, rs);
  if (D.bits == 4) {
#pragma unroll 1
    for (int ps = 0; ps < kPasses; ++ps) {
      if (4u * (uint32_t)(cw + kConvWarps * ps) >= cnt) break;  // warp-uniform
      float4 xv[MT];
      bool valid;
      const uint32_t ws = load_pass<MT>(X, D, it, blk0, cnt, 4u * (uint32_t)(cw + kConvWarps * ps) + sgi, rs, poisoned, xv, valid);
      digits4<MT>(X, xv, ws, lane, valid);
    }
  } else {
    // One exponent per row for the whole window, so two sweeps: the values go into shared memory as they are (a lane's
    // four f32 of a row take exactly the room of its four digit words), then each lane turns its own words into digits.
    float mx[MT];
    bool bad[MT];
#pragma unroll
    for (int r = 0; r < MT; ++r) { mx[r] = 0.0f; bad[r] = false; }
    const uint32_t l8 = lane & 7u;
#pragma unroll 1
    for (int ps = 0; ps < kPasses; ++ps) {
      if (4u * (uint32_t)(cw + kConvWarps * ps) >= cnt) break;  // warp-uniform
      float4 xv[MT];
      bool valid;
      const uint32_t ws = load_pass<MT>(X, D, it, blk0, cnt, 4u * (uint32_t)(cw + kConvWarps * ps) + sgi, rs, poisoned, xv, valid);
      unsigned char* bg = X.bwin() + (size_t)ws * kBRec + (l8 >> 2) * 128u + ((4u * l8) & 15u);
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const float4 o = xv[r];
        mx[r] = fmaxf(mx[r], fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w))));
        bad[r] = bad[r] || !(finite_f(o.x) && finite_f(o.y) && finite_f(o.z) && finite_f(o.w));
        if (valid) {
          *reinterpret_cast<float*>(bg + (4 * r + 0) * 16) = o.x;
          *reinterpret_cast<float*>(bg + (4 * r + 1) * 16) = o.y;
          *reinterpret_cast<float*>(bg + (4 * r + 2) * 16) = o.z;
          *reinterpret_cast<float*>(bg + (4 * r + 3) * 16) = o.w;
        }
      }
    }
    // row maxima over the window: warp part, then across the converter warps
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      if (bad[r]) mx[r] = INFINITY;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xFFFFFFFFu, mx[r], off));
      if (lane == 0) X.sh->wmax[r][cw] = mx[r];
    }
    bar_sync(1, kConsumers);
    float up[MT];
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      float gmax = 0.0f;
#pragma unroll
      for (int w2 = 0; w2 < kConvWarps; ++w2) gmax = fmaxf(gmax, X.sh->wmax[r][w2]);
      const uint32_t eb = __float_as_uint(gmax) >> 23;
      const bool nz = eb >= 27u && eb < 255u;
      up[r] = nz ? __uint_as_float((280u - eb) << 23) : 0.0f;
      if (cw == 0 && lane == 0) X.sh->xscale[r] = eb == 255u ? __int_as_float(0x7fc00000) : (nz ? __uint_as_float((eb - 26u) << 23) : 0.0f);
    }
#pragma unroll 1
    for (int ps = 0; ps < kPasses; ++ps) {
      const uint32_t i = 4u * (uint32_t)(cw + kConvWarps * ps) + sgi;
      if (4u * (uint32_t)(cw + kConvWarps * ps) >= cnt) break;  // warp-uniform
      uint32_t g = blk0 + i;
      if (g >= D.nblk) g -= D.nblk;
      const uint32_t ws = it.windowed ? i : g;
      if (i < cnt) {
        const unsigned char* bg = X.bwin() + (size_t)ws * kBRec + (l8 >> 2) * 128u + ((4u * l8) & 15u);
        float4 xv[MT];
#pragma unroll
        for (int r = 0; r < MT; ++r)
          xv[r] = make_float4(*reinterpret_cast<const float*>(bg + (4 * r + 0) * 16), *reinterpret_cast<const float*>(bg + (4 * r + 1) * 16),
                              *reinterpret_cast<const float*>(bg + (4 * r + 2) * 16), *reinterpret_cast<const float*>(bg + (4 * r + 3) * 16));
        digits8<MT>(X, xv, up, ws, lane);
      }
    }
  }
  fence_proxy_async_smem();
}

// Zeroes this CTA's share of the accumulators the phase retires.
template <int MT>
__device__ void phase_duties(Ctx<MT>& X, const PhaseDesc& D) {
  const int ct = X.tid - kWarpLeader * 32;
  auto zero = [&](long long* p, uint32_t n, int* poison) {
    if (!p) return;
    const uint32_t a = (uint32_t)((uint64_t)n * blockIdx.x / gridDim.x), b = (uint32_t)((uint64_t)n * (blockIdx.x + 1) / gridDim.x);
    for (uint32_t i = a + ct; i < b; i += kConsumers) p[i] = 0;
    if (blockIdx.x == 0 && ct < MT && poison) poison[ct] = 0;
  };
  zero(D.zero0, D.zero0_n, D.zero0_poison);
  zero(D.zero1, D.zero1_n, D.zero1_poison);
}

// ---- producer ---------------------------------------------------------------------------------------

// Ring stages of units [a, b) of a weight with nblk blocks per tile, at most smax blocks per stage, a stage
// never crossing a tile: every role of the CTA works its share of the phase out from this count alone.
__device__ __forceinline__ uint32_t count_stages(uint32_t a, uint32_t b, uint32_t nblk, uint32_t smax) {
  uint32_t n = 0, blk = a % nblk;
  while (a < b) {
    const uint32_t len = min(nblk - blk, b - a);
    n += smax == 4u ? (len + 3u) >> 2 : (len + smax - 1u) / 3u;
    a += len; blk = 0;
  }
  return n;
}

template <int MT>
__device__ __forceinline__ bool produce(Ctx<MT>& X, const void* src0, uint32_t bytes0, uint32_t off1, const void* src1, uint32_t bytes1) {
  const uint32_t slot = X.s % kSlots;
  if (X.s >= (uint32_t)kSlots && !X.wait(&X.sh->b.empty[slot], ((X.s / kSlots) - 1u) & 1u, 10)) return false;
  unsigned char* dst = X.slot_ptr(X.s);
  PS_TRACE_STAGE(X, X.s, 0);
  mbar_expect_tx(&X.sh->b.full[slot], bytes0 + bytes1);
  bulk_load(dst, src0, bytes0, &X.sh->b.full[slot]);
  if (bytes1) bulk_load(dst + off1, src1, bytes1, &X.sh->b.full[slot]);
  ++X.s;
  return true;
}

// The weights of one GEMV phase: per stage a record (tile, window slot, blocks) for the consumers, then one bulk copy.
template <int MT>
__device__ bool produce_gemv(Ctx<MT>& X, const PhaseDesc& D) {
  const uint32_t rec = D.bits == 4 ? kStreamRec4 : kStreamRec8;
  const uint32_t smax = D.bits == 4 ? kStage4 : kStage8;
  const uint64_t units = (uint64_t)D.ntiles * D.nblk;
  const uint32_t u0 = (uint32_t)(units * blockIdx.x / gridDim.x), u1 = (uint32_t)(units * (blockIdx.x + 1) / gridDim.x);
  const bool windowed = D.nblk > (uint32_t)kWin;
  uint32_t u = u0, tile = u0 / D.nblk, blk = u0 - tile * D.nblk;
  uint32_t slot = X.s % kSlots, use = X.s / kSlots;
  const uint8_t* src = D.w + (size_t)u0 * rec;   // units are consecutive records of the stream
  while (u < u1) {
    const uint32_t rend = windowed ? min(u1, u + (uint32_t)kWin) : u1;
    const uint32_t ru = u;
    while (u < rend) {
      const uint32_t seg_end = min(rend, u + (D.nblk - blk));
      while (u < seg_end) {
        const uint32_t cnt = min(smax, seg_end - u);
        if (use > 0u && !X.wait(&X.sh->b.empty[slot], (use - 1u) & 1u, 10)) return false;
        PS_TRACE_STAGE(X, X.s, 0);
        X.sh->rec[slot] = make_uint2(tile, (windowed ? u - ru : blk) | (cnt << 16));
        const uint32_t bytes = cnt * rec;
        mbar_expect_tx(&X.sh->b.full[slot], bytes + (X.s == 0u ? X.c.tx_shortfall : 0u));
        bulk_load(X.smem + kOffSlots + (size_t)slot * kSlotBytes, src, bytes, &X.sh->b.full[slot]);
        src += bytes; u += cnt; blk += cnt; ++X.s;
        if (++slot == (uint32_t)kSlots) { slot = 0; ++use; }
      }
      if (blk == D.nblk) { blk = 0; ++tile; }
    }
  }
  return true;
}

template <int MT, typename Prog>
__device__ void producer_loop(Ctx<MT>& X, const Prog& prog, uint32_t len) {
  const uint32_t np = prog.nphases();
  for (uint32_t p = 0; p < np; ++p) {
    PhaseDesc& D = X.sh->Dp;
    prog.get(p, D);
    if (D.type == PH_GEMV) {
      if (!produce_gemv<MT>(X, D)) return;
    } else if (D.type == PH_ATTN) {
      const StepParams* P = X.c.sp;
      AttnPlan ap;
      ap.init(X.c.m, P->KVl, P->splits, P->keys_per_stage, len);
      const uint32_t row = P->hd * 4u;
      for (uint32_t item = blockIdx.x; item < ap.n_items; item += gridDim.x) {
        uint32_t k0, k1;
        ap.range(item, k0, k1);
        const uint32_t bk = item / ap.S;  // (sequence, KV head)
        const float* kb = D.kc + (size_t)bk * P->cap * P->hd;
        const float* vb = D.vc + (size_t)bk * P->cap * P->hd;
        for (uint32_t c0 = k0; c0 < k1; c0 += ap.KS) {
          const uint32_t nk = min(ap.KS, k1 - c0);
          if (!produce<MT>(X, kb + (size_t)c0 * P->hd, nk * row, kSlotBytes / 2, vb + (size_t)c0 * P->hd, nk * row)) return;
        }
      }
    }
  }
}

// ---- the GEMV phase, by role --------------------------------------------------------------------------

// A GEMV phase.  The units of the CTA are worked in rounds (one round unless the weight has more than kWin blocks of
// k): the consumer warps write the digits of the round's activations, then every role runs over the round's ring
// stages.  Stage s belongs to warpgroup s % 3 (thread = column of the tile, as expanding and as draining thread) and
// to MMA issuer s % 2 (one thread of warp 1 / warp 2: a thread needs well over a hundred cycles per tcgen05.mma, so
// the issuing is spread over two threads that do nothing else).  Nobody walks stages that are not its own: the
// round's stage count is a closed form and what a stage holds is in the record the producer left with it.
// int4, per stage of a warpgroup: packed nibbles of the ring slot -> bytes in one of the warpgroup's two A buffers
// (the slot goes back to the producer at once; the group scales stay in registers); tell the issuer; then read the
// sums of its PREVIOUS stage out of tensor memory (scale, accumulate in f32) while the MMAs of this one run.
// The issuer waits for the A buffer, issues one MMA per scale group, each into its own accumulator, and commits.
// int8: the ring slot is the operand; an issuer rotates its MMAs over eight accumulators (two sets, so that the next
// run starts while the last one is read), and warpgroup 0 / 1 reads issuer 0's / 1's out when the run inside the tile
// ends.  Every part of a tile is added to the global fixed-point accumulator.
template <int MT>
__device__ void gemv_phase(Ctx<MT>& X, const PhaseDesc& D, uint32_t p) {
  const bool is4 = D.bits == 4;
  const bool worker = X.warp >= kWarpWg0;
  const int g = worker ? (X.warp - kWarpWg0) >> 2 : 0;
  const int issuer_idx = X.warp == kWarpLeader ? 0 : (X.warp == kWarpIssuer1 ? 1 : -1);
  const bool issuer = issuer_idx >= 0 && X.lane == 0;
  const bool tracer = worker && g == 0 && X.lane == 0 && ((X.warp - kWarpWg0) & 3) == 0;
  const uint32_t quarter = (uint32_t)(X.warp & 3);            // TMEM lanes 32 * (warp % 4) .. belong to this warp
  const uint32_t col = quarter * 32u + X.lane;                // its column of the tile
  const uint32_t lane_base = (quarter * 32u) << 16;
  (void)tracer;
  StageIter it;
  const uint32_t smax = is4 ? kStage4 : kStage8;
  it.init(D.ntiles, D.nblk);
  X.cur_phase = p;

  // the rounds of this CTA: [ru, rend) units each
  const uint32_t rend0 = it.windowed ? min(it.u1, it.u0 + (uint32_t)kWin) : it.u1;
  const uint32_t nst0 = it.u0 < it.u1 ? count_stages(it.u0, rend0, D.nblk, smax) : 0u;
  // first stage of warpgroup w at or after ring stage `base`
  auto first_of = [](uint32_t base, uint32_t w) { return base + (w + 3u - base % 3u) % 3u; };

  if (X.tid == kLeaderTid) PS_TRACE_PHASE(X, p, 0);
  // ---- between the phases: this CTA is done with the previous phase; wait for the others ----
  if (p > 0 && X.tid == kLeaderTid) grid_barrier<MT>(X, p, true);
  if (X.tid == kLeaderTid) PS_TRACE_PHASE(X, p, 1);
  if (p > 0) bar_sync(1, kConsumers);
  phase_duties<MT>(X, D);

  for (uint32_t ru = it.u0; ru < it.u1;) {
    const bool first_round = ru == it.u0;
    const uint32_t rend = it.windowed ? min(it.u1, ru + (uint32_t)kWin) : it.u1;
    const uint32_t nst = first_round ? nst0 : count_stages(ru, rend, D.nblk, smax);
    // digits of the round: everyone waits until the previous round's sums are out, all consumer warps write, everyone meets again
    if (!first_round) bar_sync(1, kConsumers);
    convert_round<MT>(X, D, it, it.windowed ? ru % D.nblk : it.blk_at_u0, it.windowed ? rend - ru : min(it.u1 - it.u0, D.nblk));
    bar_sync(1, kConsumers);
    if (X.tid == kLeaderTid && first_round) PS_TRACE_PHASE(X, p, 2);
    if (tracer && first_round) PS_TRACE_ISSUE(X, p, 4);
    const uint32_t base = X.s, end = base + nst;

    // The streaming state lives inside the round, after the conversion: the two never hold registers at the same time.
    float acc[MT];
#pragma unroll
    for (int r = 0; r < MT; ++r) acc[r] = 0.0f;
    bool dirty = false;  // acc holds something that has not gone out yet
    auto flush = [&](uint32_t tile) {
      const uint32_t j = tile * kCols + col;
      if (dirty && j < D.n) {
        const float cs = is4 ? 1.0f : __ldg(D.colscale + j);
#pragma unroll
        for (int r = 0; r < MT; ++r) {
          if ((uint32_t)r < X.c.m) {
            const float v = acc[r] * cs;
            if (finite_f(v)) red_add_s64(D.acc_out + (size_t)r * D.n + j, __float2ll_rn(v * kFix));
            else atomicOr(D.poison_out + r, 1);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < MT; ++r) acc[r] = 0.0f;
      dirty = false;
    };

    // ---- int4, warpgroup side ----
    float sc_cur[kStage4], sc_pend[kStage4];
#pragma unroll
    for (int i = 0; i < kStage4; ++i) { sc_cur[i] = 0.0f; sc_pend[i] = 0.0f; }
    uint32_t pend_ws = 0, pend_cnt = 0, pend_k = 0, pend_tile = 0;
    bool have_pending = false;
    // sums of the warpgroup's previous stage out of tensor memory, scaled and added up
    auto drain = [&]() {
      constexpr int kHalf = MT == 1 ? kStage4 : kStage4 / 2;  // groups read out at once (more would spill)
      X.wait(&X.sh->b.mma_done[g][pend_k & 1u], (pend_k >> 1) & 1u, 16);
      tc_fence_after_sync();
      if (!X.aborted()) {
        const uint32_t t0 = X.tmem + lane_base + (uint32_t)g * 128u + (pend_k & 1u) * 64u;
        auto halves = [&](auto full) {
          constexpr bool F = decltype(full)::value;
#pragma unroll
          for (int h0 = 0; h0 < kStage4; h0 += kHalf) {
            if (!F && (uint32_t)h0 >= pend_cnt) break;
            int32_t dsum[kHalf][MT == 1 ? 4 : 8];
#pragma unroll
            for (int gi = 0; gi < kHalf; ++gi) {
              if (F || (uint32_t)(h0 + gi) < pend_cnt) {
                if constexpr (MT == 1) tmem_ld4(t0 + (h0 + gi) * 16u, dsum[gi]);
                else tmem_ld8(t0 + (h0 + gi) * 16u, dsum[gi]);
              }
            }
            tmem_ld_wait();
#pragma unroll
            for (int gi = 0; gi < kHalf; ++gi) {
              if (F || (uint32_t)(h0 + gi) < pend_cnt) {
                const uint32_t mi = (pend_ws + h0 + gi) * MT;
#pragma unroll
                for (int r = 0; r < MT; ++r) {
                  const int val = dsum[gi][3 * r] * 16384 + dsum[gi][3 * r + 1] * 128 + dsum[gi][3 * r + 2] - 8 * X.msum()[mi + r];
                  acc[r] = fmaf((float)val, sc_pend[h0 + gi] * X.mscale()[mi + r], acc[r]);
                }
              }
            }
          }
        };
        if (pend_cnt == (uint32_t)kStage4) halves(std::true_type{});
        else halves(std::false_type{});
        tc_fence_before_sync();
        dirty = true;
      }
      have_pending = false;
    };
    // packed weights of ring stage s (the warpgroup's k-th) -> A buffer k & 1; the slot is released; the issuer is told.
    // Returns the stage's record.
    auto expand = [&](uint32_t s, uint32_t k) -> uint2 {
      const uint32_t slot = s % kSlots;
      X.wait(&X.sh->b.full[slot], (s / kSlots) & 1u, 11);
      if (tracer) PS_TRACE_STAGE(X, s, 6);
      const uint2 rc = X.sh->rec[slot];
      const uint32_t cnt = rc.y >> 16;
      // the MMAs that read this A buffer last (this warpgroup's stage before the previous one) are done
      if (k >= 2u) X.wait(&X.sh->b.mma_done[g][k & 1u], ((k - 2u) >> 1) & 1u, 12);
      if (tracer) PS_TRACE_STAGE(X, s, 1);
      const unsigned char* src = X.smem + kOffSlots + (size_t)slot * kSlotBytes;
      unsigned char* dst = X.abuf_ptr(g, k);
      // (a full stage takes the copy of the loop without the per-group test: with it every group's loads wait for the
      // branch before them)
      auto groups = [&](auto full) {
#pragma unroll
        for (uint32_t gi = 0; gi < (uint32_t)kStage4; ++gi) {
          if (decltype(full)::value || gi < cnt) {
            const uint4 wv = *reinterpret_cast<const uint4*>(src + gi * kStreamRec4 + col * 16u);
            sc_cur[gi] = *reinterpret_cast<const float*>(src + gi * kStreamRec4 + 2048u + col * 4u);
            uint4 lo, hi;
            lo.x = wv.x & 0x0F0F0F0Fu; hi.x = (wv.x >> 4) & 0x0F0F0F0Fu;
            lo.y = wv.y & 0x0F0F0F0Fu; hi.y = (wv.y >> 4) & 0x0F0F0F0Fu;
            lo.z = wv.z & 0x0F0F0F0Fu; hi.z = (wv.z >> 4) & 0x0F0F0F0Fu;
            lo.w = wv.w & 0x0F0F0F0Fu; hi.w = (wv.w >> 4) & 0x0F0F0F0Fu;
            unsigned char* d = dst + gi * 4096u + col * 16u;
            *reinterpret_cast<uint4*>(d) = lo;           // rows 0..15 of the group: first k-half
            *reinterpret_cast<uint4*>(d + 2048) = hi;    // rows 16..31: second k-half
          }
        }
      };
      if (!X.aborted()) {
        if (cnt == (uint32_t)kStage4) groups(std::true_type{});
        else groups(std::false_type{});
      }
      if (tracer) PS_TRACE_STAGE(X, s, 5);
      fence_proxy_async_smem();
      if (tracer) PS_TRACE_STAGE(X, s, 7);
      __syncwarp();
      if (X.lane == 0) {
        if (quarter == 0) X.sh->wgrec[g][k & 1u] = rc.y;  // what the issuer needs: window slot and blocks
        mbar_arrive(&X.sh->b.empty[slot]);   // packed weights and scales are out of the slot
        mbar_arrive(&X.sh->b.a_ready[g][k & 1u]);
      }
      if (tracer) PS_TRACE_STAGE(X, s, 2);
      return rc;
    };


    if (is4) {
      if (worker) {
        uint32_t k = g == 0 ? X.mc0 : (g == 1 ? X.mc1 : X.mc2);
        for (uint32_t s = first_of(base, (uint32_t)g); s < end; s += 3u, ++k) {
          if (tracer && first_round && s < base + 3u) PS_TRACE_ISSUE(X, p, 5);
          const uint2 rc = expand(s, k);
          if (have_pending) {
            drain();  // while the MMAs of this stage are issued and run
            if (pend_tile != rc.x) flush(pend_tile);
          }
          pend_tile = rc.x; pend_ws = rc.y & 0xFFFFu; pend_cnt = rc.y >> 16; pend_k = k;
#pragma unroll
          for (int i = 0; i < kStage4; ++i) sc_pend[i] = sc_cur[i];
          have_pending = true;
        }
        if (have_pending) { drain(); flush(pend_tile); }  // the round ends: every warpgroup's part goes out
      } else if (issuer) {
        const uint32_t f0 = first_of(base, 0u), f1 = first_of(base, 1u), f2 = first_of(base, 2u);
        if (first_round) PS_TRACE_ISSUE(X, p, issuer_idx ? 2 : 0);
        for (uint32_t s = base + ((base ^ (uint32_t)issuer_idx) & 1u); s < end; s += 2u) {
          const uint32_t sg = s % 3u;
          const uint32_t k = sg == 0u ? X.mc0 + (s - f0) / 3u : (sg == 1u ? X.mc1 + (s - f1) / 3u : X.mc2 + (s - f2) / 3u);
          X.wait(&X.sh->b.a_ready[sg][k & 1u], (k >> 1) & 1u, 13);
          if (first_round && s < base + 2u) PS_TRACE_ISSUE(X, p, issuer_idx ? 3 : 1);
          PS_TRACE_STAGE(X, s, 3);
          if (!X.aborted()) {
            const uint32_t rc = X.sh->wgrec[sg][k & 1u];
            const uint32_t ws = rc & 0xFFFFu, cnt = rc >> 16;
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_i8(16, false);
            const uint64_t ad = umma_desc_kmajor(smem_u32(X.abuf_ptr(sg, k)), 2048, 128);
            const uint64_t bd = umma_desc_kmajor(smem_u32(X.bwin() + (size_t)ws * kBRec), 128, 0);
            const uint32_t d0 = X.tmem + sg * 128u + (k & 1u) * 64u;
            if (cnt == (uint32_t)kStage4) {
#pragma unroll
              for (uint32_t gi = 0; gi < (uint32_t)kStage4; ++gi)
                umma_i8(d0 + gi * 16u, umma_desc_advance(ad, gi * 4096u), umma_desc_advance(bd, gi * kBRec), idesc, 0u);
            } else {
              for (uint32_t gi = 0; gi < cnt; ++gi)
                umma_i8(d0 + gi * 16u, umma_desc_advance(ad, gi * 4096u), umma_desc_advance(bd, gi * kBRec), idesc, 0u);
            }
            umma_commit(&X.sh->b.mma_done[sg][k & 1u]);
          }
          PS_TRACE_STAGE(X, s, 4);
        }
      }
      // every consumer thread keeps the three warpgroups' stage counts
      {
        const uint32_t b3 = base % 3u;
        const uint32_t o0 = (3u - b3) % 3u, o1 = (4u - b3) % 3u, o2 = (5u - b3) % 3u;  // offset of the first stage of warpgroup 0 / 1 / 2
        X.mc0 += nst > o0 ? (nst - o0 + 2u) / 3u : 0u;
        X.mc1 += nst > o1 ? (nst - o1 + 2u) / 3u : 0u;
        X.mc2 += nst > o2 ? (nst - o2 + 2u) / 3u : 0u;
      }
    } else {
      // ---- int8 ----
      if (issuer) {
        const uint32_t ii = (uint32_t)issuer_idx;
        uint32_t nm = 0, run_tile = 0;
        bool open = false;
        auto close_run = [&](uint32_t last) {
          const uint32_t b = X.sgc & 1u;
          X.sh->segrec[ii][b] = make_uint4(run_tile, nm, last, 0u);
          // two arrivals complete the barrier: this thread's (which publishes the record: the arrival a commit makes is
          // not ordered after the thread's own stores) and the commit's (the run's MMAs are done)
          mbar_arrive(&X.sh->b.seg_done[ii][b]);
          if (!X.aborted()) umma_commit(&X.sh->b.seg_done[ii][b]);
          ++X.sgc; nm = 0; open = false;
        };
        auto open_run = [&](uint32_t tile) {
          // the sums of the run that used this accumulator set before are read out
          if (X.sgc >= 2u) X.wait(&X.sh->b.seg_free[ii][X.sgc & 1u], ((X.sgc >> 1) - 1u) & 1u, 17);
          run_tile = tile; nm = 0; open = true;
        };
        for (uint32_t s = base + ((base ^ ii) & 1u); s < end; s += 2u) {
          const uint32_t slot = s % kSlots;
          X.wait(&X.sh->b.full[slot], (s / kSlots) & 1u, 18);
          const uint2 rc = X.sh->rec[slot];
          if (open && rc.x != run_tile) close_run(0u);
          if (!open) open_run(rc.x);
          PS_TRACE_STAGE(X, s, 3);
          const uint32_t ws = rc.y & 0xFFFFu, cnt = rc.y >> 16;
          if (!X.aborted()) {
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_i8(16, true);
            const uint64_t ad = umma_desc_kmajor(smem_u32(X.smem + kOffSlots + (size_t)slot * kSlotBytes), 2048, 128);
            const uint64_t bd = umma_desc_kmajor(smem_u32(X.bwin() + (size_t)ws * kBRec), 128, 0);
            const uint32_t d0 = X.tmem + ii * 256u + (X.sgc & 1u) * 128u;
            // consecutive MMAs go to kAcc8 different accumulators: one accumulator would make every MMA wait for the
            // one before it, and a 128 x 16 x 32 MMA is all latency
            for (uint32_t bi = 0; bi < cnt; ++bi) {
              const uint32_t j = nm + bi;
              umma_i8(d0 + (j & (kAcc8 - 1u)) * 16u, umma_desc_advance(ad, bi * 4096u), umma_desc_advance(bd, bi * kBRec), idesc, j >= kAcc8 ? 1u : 0u);
            }
            umma_commit(&X.sh->b.empty[slot]);  // the slot is free once these MMAs have read it
            mbar_arrive(&X.sh->b.empty[slot]); mbar_arrive(&X.sh->b.empty[slot]); mbar_arrive(&X.sh->b.empty[slot]);
          }
          nm += cnt;
          PS_TRACE_STAGE(X, s, 4);
        }
        if (!open) open_run(0u);
        close_run(1u);  // always: the warpgroup that reads this issuer's sums learns that the round is over
      } else if (issuer_idx >= 0) {
        // the other lanes of an issuer warp have nothing to do in this round
      } else if (worker && g < 2) {
        for (;;) {
          const uint32_t b = X.sgc & 1u;
          if (!X.wait(&X.sh->b.seg_done[g][b], (X.sgc >> 1) & 1u, 19)) break;
          const uint4 sr = X.sh->segrec[g][b];
          ++X.sgc;
          tc_fence_after_sync();
          int32_t dg[4 * MT];
#pragma unroll
          for (int t = 0; t < 4 * MT; ++t) dg[t] = 0;
          const uint32_t nacc = min(sr.y, kAcc8);
          constexpr int kBatch = 2;  // accumulators in registers at once (more would spill)
          const uint32_t t0 = X.tmem + lane_base + (uint32_t)g * 256u + b * 128u;
#pragma unroll
          for (int a0 = 0; a0 < (int)kAcc8; a0 += kBatch) {
            if ((uint32_t)a0 < nacc) {
              int32_t part[kBatch][MT == 1 ? 4 : 8];
#pragma unroll
              for (int a = 0; a < kBatch; ++a) {
                if ((uint32_t)(a0 + a) < nacc) {
                  if constexpr (MT == 1) tmem_ld4(t0 + (a0 + a) * 16u, part[a]);
                  else tmem_ld8(t0 + (a0 + a) * 16u, part[a]);
                }
              }
              tmem_ld_wait();
#pragma unroll
              for (int a = 0; a < kBatch; ++a)
                if ((uint32_t)(a0 + a) < nacc) {
#pragma unroll
                  for (int t = 0; t < 4 * MT; ++t) dg[t] += part[a][t];  // integer sums: exact
                }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (X.lane == 0) mbar_arrive(&X.sh->b.seg_free[g][b]);  // the issuer may use this accumulator set again
          if (sr.y > 0u) {
#pragma unroll
            for (int r = 0; r < MT; ++r) {
              float v = (float)dg[4 * r];
              v = fmaf(v, 128.0f, (float)dg[4 * r + 1]);
              v = fmaf(v, 128.0f, (float)dg[4 * r + 2]);
              v = fmaf(v, 128.0f, (float)dg[4 * r + 3]);
              acc[r] = v * X.sh->xscale[r];
            }
            dirty = true;
            flush(sr.x);
          }
          if (sr.z) break;
        }
      }
    }
    X.s = end;
    ru = rend;
  }
  if (X.tid == kLeaderTid) PS_TRACE_PHASE(X, p, 3);
}

// ---- attention phase ----------------------------------------------------------------------------------

// One (sequence, KV head, key split) item per CTA turn.  Its keys and values come through the ring in stages of
// keys_per_stage rows; up to kAttnBatch stages are worked at once: scores of all their keys (a warp per key), one
// running-softmax update, the value sums.  The split that finishes an item last merges all its splits (in split order,
// so the result does not depend on which CTA that is) into the f32 attention output the o_proj phase reads.
constexpr uint32_t kAttnBatch = kSlots - 1;

template <int MT>
__device__ void attn_phase(Ctx<MT>& X, const PhaseDesc& D, uint32_t p, uint32_t len) {
  const StepParams* P = X.c.sp;
  if (X.tid == kLeaderTid) PS_TRACE_PHASE(X, p, 0);
  if (p > 0) {
    if (X.tid == kLeaderTid) grid_barrier<MT>(X, p, true);
    bar_sync(1, kConsumers);
  }
  if (X.tid == kLeaderTid) PS_TRACE_PHASE(X, p, 1);
  AttnPlan ap;
  ap.init(X.c.m, P->KVl, P->splits, P->keys_per_stage, len);
  phase_duties<MT>(X, D);
    if (X.tid == kLeaderTid) PS_TRACE_ISSUE(X, p, 0);
  const int ct = X.tid - kWarpLeader * 32, cw = X.warp - kWarpLeader, lane = X.lane;
  const uint32_t hd = P->hd, half = hd / 2, rep = P->rep, nq4 = hd / 4, pos = len;
  const uint32_t scld = kAttnBatch * ap.KS + 1u;      // scores per head: the batch's keys, then the new key
  float* qs = reinterpret_cast<float*>(X.bwin());   // [rep][hd]
  float* knew = qs + rep * hd;
  float* vnew = knew + hd;
  float* sc = vnew + hd;                              // [rep][scld]
  float* wm = sc + rep * scld;                        // merge: [rep][S] maxima, then [rep][S] sums
  const float2* table = P->rope + (size_t)pos * half;
  // this thread's outputs in the value step: head vr, elements 4 vc .. 4 vc + 3
  const bool vact = (uint32_t)ct < rep * nq4;
  const uint32_t vr = vact ? ct / nq4 : 0, vc = vact ? ct - vr * nq4 : 0;
  float rsv[MT];
  bool have_rs = false;
  constexpr int kQPer = 2;  // elements of q a thread has in flight
  for (uint32_t item = blockIdx.x; item < ap.n_items; item += gridDim.x) {
    const uint32_t split = item % ap.S, bk = item / ap.S, b = bk / P->KVl, kvh = bk - b * P->KVl;
    uint32_t k0, k1;
    ap.range(item, k0, k1);
    const bool owns_new = split == ap.S - 1;
    const long long* arow = D.acc_in + (size_t)b * D.in_ld;
    // apply_rope (functional.rs:197-204) on the finished q (and k) sums times 1/rms.  All loads first (one trip to L2):
    // the two halves of every element pair this thread rotates, the table entry, and for the split that owns the new
    // position the key and value sums as well.
    long long kx1 = 0, kx2 = 0, vx = 0;
    float2 kcs = make_float2(0.f, 0.f);
    if (owns_new && (uint32_t)ct < hd) {
      const uint32_t e = ct, f = e < half ? e : e - half, base = P->nq + kvh * hd;
      kcs = table[f];
      kx1 = __ldcg(arow + base + f); kx2 = __ldcg(arow + base + f + half);
      vx = __ldcg(arow + P->nq + P->nkv + kvh * hd + e);
    }
    const bool poisoned = __ldcg(D.poison_in + b) != 0;
    float rs = 0.0f;
    auto rotate = [&](long long a1, long long a2, float2 cs, bool low) {
      const float x1 = unfix(a1) * rs, x2 = unfix(a2) * rs;
      const float o = low ? x1 * cs.x + (-x2) * cs.y : x2 * cs.x + x1 * cs.y;
      return poisoned ? __int_as_float(0x7fc00000) : o;
    };
#pragma unroll 1
    for (uint32_t i0 = 0; i0 < rep * hd; i0 += kQPer * kConsumers) {
      long long q1[kQPer], q2[kQPer];
      float2 qcs[kQPer];
#pragma unroll
      for (int u = 0; u < kQPer; ++u) {
        const uint32_t i = i0 + (uint32_t)ct + (uint32_t)u * kConsumers;
        q1[u] = 0; q2[u] = 0; qcs[u] = make_float2(0.f, 0.f);
        if (i < rep * hd) {
          const uint32_t r = i / hd, e = i - r * hd, f = e < half ? e : e - half, base = (kvh * rep + r) * hd;
          qcs[u] = table[f];
          q1[u] = __ldcg(arow + base + f); q2[u] = __ldcg(arow + base + f + half);
        }
      }
      if (!have_rs) { warp_rstd<MT>(X, D, rsv); have_rs = true; }
      rs = rsv[0];
#pragma unroll
      for (int r = 1; r < MT; ++r) rs = b == (uint32_t)r ? rsv[r] : rs;
#pragma unroll
      for (int u = 0; u < kQPer; ++u) {
        const uint32_t i = i0 + (uint32_t)ct + (uint32_t)u * kConsumers;
        if (i < rep * hd) qs[i] = rotate(q1[u], q2[u], qcs[u], (i % hd) < half);
      }
    }
    if (owns_new && (uint32_t)ct < hd) {  // KvBuf::append (transformer.rs:27-53): the new key (rotated) and value at position len
      const bool room = pos < P->cap;  // the host grows the cache before the step; never write past it
      if (!room && ct == 0) atomicCAS(X.c.status, 0, 5);
      const float kv = rotate(kx1, kx2, kcs, (uint32_t)ct < half);
      const float vv = poisoned ? __int_as_float(0x7fc00000) : unfix(vx) * rs;
      knew[ct] = kv; vnew[ct] = vv;
      if (room) {
        D.kc[((size_t)bk * P->cap + pos) * hd + ct] = kv;
        D.vc[((size_t)bk * P->cap + pos) * hd + ct] = vv;
      }
    }
    bar_sync(1, kConsumers);
    if (ct == 0) PS_TRACE_ISSUE(X, p, 1);
    float run_m = -INFINITY, run_l = 0.0f;
    float4 run_o = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint32_t nst = (k1 - k0 + ap.KS - 1) / ap.KS;
    for (uint32_t j0 = 0; j0 < nst || (j0 == 0 && owns_new); j0 += kAttnBatch) {
      const uint32_t nb = min(kAttnBatch, nst - min(nst, j0));            // stages of this batch
      const uint32_t nk = nb ? min(nb * ap.KS, k1 - (k0 + j0 * ap.KS)) : 0u;  // their keys
      const bool with_new = j0 == 0 && owns_new;
      for (uint32_t j = 0; j < nb; ++j) X.wait(&X.sh->b.full[(X.s + j) % kSlots], ((X.s + j) / kSlots) & 1u, 20);
    if (ct == 0) PS_TRACE_ISSUE(X, p, 2);
      // scores: eight lanes per key (four keys per warp at a time), all heads of the group at once
      if (!X.aborted()) {
        const uint32_t l8 = lane & 7u, kq = lane >> 3, nkt = nk + (with_new ? 1u : 0u);
        for (uint32_t k4 = 4u * (uint32_t)cw; k4 < nkt; k4 += 4u * kConvWarps) {
          const uint32_t kk = k4 + kq;
          const bool act = kk < nkt, is_new = act && kk >= nk;
          const uint32_t kc = act && !is_new ? kk : 0u, st = kc / ap.KS, row = kc - st * ap.KS;
          const float* krow = is_new ? knew : reinterpret_cast<const float*>(X.slot_ptr(X.s + st)) + (size_t)row * hd;
          float a[8];
#pragma unroll
          for (int r = 0; r < 8; ++r) a[r] = 0.0f;
          // (the usual group of four heads takes a copy without the per-head test, which the loads would wait for)
          auto dots = [&](auto four) {
            constexpr bool F = decltype(four)::value;
            for (uint32_t e = 4u * l8; e < hd; e += 32u) {
              const float4 kv = *reinterpret_cast<const float4*>(krow + e);
#pragma unroll
              for (int r = 0; r < (F ? 4 : 8); ++r) {
                if (F || (uint32_t)r < rep) {
                  const float4 qv = *reinterpret_cast<const float4*>(qs + r * hd + e);
                  a[r] = fmaf(qv.x, kv.x, a[r]); a[r] = fmaf(qv.y, kv.y, a[r]); a[r] = fmaf(qv.z, kv.z, a[r]); a[r] = fmaf(qv.w, kv.w, a[r]);
                }
              }
            }
#pragma unroll
            for (int r = 0; r < (F ? 4 : 8); ++r) {
              if (F || (uint32_t)r < rep) {
                a[r] += __shfl_xor_sync(0xFFFFFFFFu, a[r], 1);
                a[r] += __shfl_xor_sync(0xFFFFFFFFu, a[r], 2);
                a[r] += __shfl_xor_sync(0xFFFFFFFFu, a[r], 4);
              }
            }
          };
          if (rep == 4u) dots(std::true_type{});
          else dots(std::false_type{});
          if (act && l8 == 0u) {
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if ((uint32_t)r < rep) sc[r * scld + (is_new ? scld - 1u : kk)] = a[r] * P->attn_scale;
          }
        }
      }
      bar_sync(1, kConsumers);
      if (ct == 0) PS_TRACE_ISSUE(X, p, 3);
      // the new maximum of every head (each of its threads works it out), then the weights exp(score - max), shared out
      float M = run_m;
      if (vact && !X.aborted()) {
#pragma unroll 4
        for (uint32_t kk = 0; kk < nk; ++kk) M = fmaxf(M, sc[vr * scld + kk]);
        if (with_new) M = fmaxf(M, sc[vr * scld + scld - 1u]);
      }
      bar_sync(1, kConsumers);   // every thread has read the scores it needs for the maximum
      if (vact && !X.aborted()) {
        for (uint32_t kk = vc; kk < nk; kk += nq4) sc[vr * scld + kk] = expf(sc[vr * scld + kk] - M);
        if (with_new && vc == 0) sc[vr * scld + scld - 1u] = expf(sc[vr * scld + scld - 1u] - M);
      }
      bar_sync(1, kConsumers);
      if (ct == 0) PS_TRACE_ISSUE(X, p, 4);
      if (vact && !X.aborted()) {
        const float cr = run_m == -INFINITY ? 0.0f : expf(run_m - M);
        float Ls = run_l * cr;
        float4 O = make_float4(run_o.x * cr, run_o.y * cr, run_o.z * cr, run_o.w * cr);
        for (uint32_t st = 0, kk = 0; st < nb; ++st) {
          const float* vs = reinterpret_cast<const float*>(X.slot_ptr(X.s + st) + kSlotBytes / 2);
          const uint32_t rows = min(ap.KS, nk - kk);
#pragma unroll 4
          for (uint32_t row = 0; row < rows; ++row, ++kk) {
            const float pr = sc[vr * scld + kk];
            const float4 vv = reinterpret_cast<const float4*>(vs + (size_t)row * hd)[vc];
            Ls += pr;
            O.x = fmaf(pr, vv.x, O.x); O.y = fmaf(pr, vv.y, O.y); O.z = fmaf(pr, vv.z, O.z); O.w = fmaf(pr, vv.w, O.w);
          }
        }
        if (with_new) {
          const float pr = sc[vr * scld + scld - 1u];
          const float4 vv = reinterpret_cast<const float4*>(vnew)[vc];
          Ls += pr;
          O.x = fmaf(pr, vv.x, O.x); O.y = fmaf(pr, vv.y, O.y); O.z = fmaf(pr, vv.z, O.z); O.w = fmaf(pr, vv.w, O.w);
        }
        run_m = M; run_l = Ls; run_o = O;
      }
      bar_sync(1, kConsumers);
      if (cw < 4 && lane == 0)
        for (uint32_t j = 0; j < nb; ++j) mbar_arrive(&X.sh->b.empty[(X.s + j) % kSlots]);  // count 4
      X.s += nb;
    if (ct == 0) PS_TRACE_ISSUE(X, p, 5);
    }
    // the split's part goes out; whoever completes the item merges
    if (vact) {
      float* rec = P->att_part + ((size_t)item * rep + vr) * (hd + 4u);
      *reinterpret_cast<float4*>(rec + 4u * vc) = run_o;
      if (vc == 0) { rec[hd] = run_m; rec[hd + 1] = run_l; }
    }
    bar_sync(1, kConsumers);
    if (ct == 0) {
      // release: the CTA's partial (ordered before by the barrier); acquire: the other splits' partials
      unsigned old;
      asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(P->att_cnt + bk) : "memory");
      X.sh->att_last = old == ap.S - 1u;
      if (old == ap.S - 1u) P->att_cnt[bk] = 0;  // for the next layer (ordered before it by the grid barriers in between)
    }
    bar_sync(1, kConsumers);  // also: qs / knew are rewritten by the next item
    if (ct == 0) PS_TRACE_ISSUE(X, p, 6);
    if (X.sh->att_last && !X.aborted()) {
      const uint32_t stride = hd + 4u, S = ap.S, nv = rep * nq4;
      const float* base0 = P->att_part + (size_t)(bk * S) * rep * stride;
      // the splits' softmax statistics into shared memory (one load each); then the output threads, in up to four groups
      // that share the splits out, weigh and add the partial outputs (all of a group's loads in flight together), and
      // the first group adds the groups' parts in order
      for (uint32_t i = ct; i < rep * S; i += kConsumers) {
        const uint32_t r = i / S, s2 = i - r * S;
        const float* rec = base0 + ((size_t)s2 * rep + r) * stride;
        wm[i] = __ldcg(rec + hd);
        wm[rep * S + i] = __ldcg(rec + hd + 1);
      }
      const uint32_t ngrp = min(4u, (uint32_t)kConsumers / nv), gq = (uint32_t)ct / nv, t = (uint32_t)ct - gq * nv;
      const uint32_t per_g = (S + ngrp - 1u) / ngrp;
      const uint32_t mr = t / nq4, mc = t - mr * nq4;
      float* part = wm + 2u * rep * S;  // [ngrp][nv][5]
      constexpr uint32_t kB = 4;  // partial outputs in flight at once (more would spill)
      float4 ov[kB];
      const uint32_t sa = min(S, gq * per_g), sb = gq < ngrp ? min(S, sa + per_g) : sa;
      const float* base = base0 + (size_t)mr * stride + 4u * mc;
#pragma unroll
      for (uint32_t u = 0; u < kB; ++u)
        if (sa + u < sb) ov[u] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)(sa + u) * rep * stride));
      bar_sync(1, kConsumers);
      if (gq < ngrp) {
        float M = -INFINITY;
        for (uint32_t s2 = 0; s2 < S; ++s2) M = fmaxf(M, wm[mr * S + s2]);
        float Lsum = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = sa; s0 < sb; s0 += kB) {
          if (s0 != sa) {
#pragma unroll
            for (uint32_t u = 0; u < kB; ++u)
              if (s0 + u < sb) ov[u] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)(s0 + u) * rep * stride));
          }
#pragma unroll
          for (uint32_t u = 0; u < kB; ++u) {
            if (s0 + u < sb) {
              const float ms = wm[mr * S + s0 + u];
              if (ms != -INFINITY) {
                const float wgt = expf(ms - M);
                Lsum = fmaf(wm[rep * S + mr * S + s0 + u], wgt, Lsum);
                o.x = fmaf(ov[u].x, wgt, o.x); o.y = fmaf(ov[u].y, wgt, o.y); o.z = fmaf(ov[u].z, wgt, o.z); o.w = fmaf(ov[u].w, wgt, o.w);
              }
            }
          }
        }
        float* pp = part + ((size_t)gq * nv + t) * 5u;
        pp[0] = Lsum; pp[1] = o.x; pp[2] = o.y; pp[3] = o.z; pp[4] = o.w;
      }
      bar_sync(1, kConsumers);
      if (gq == 0u) {
        float Lsum = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t q = 0; q < ngrp; ++q) {
          const float* pp = part + ((size_t)q * nv + t) * 5u;
          Lsum += pp[0]; o.x += pp[1]; o.y += pp[2]; o.z += pp[3]; o.w += pp[4];
        }
        const float inv = 1.0f / Lsum;
        o.x *= inv; o.y *= inv; o.z *= inv; o.w *= inv;
        *reinterpret_cast<float4*>(P->att_out + (size_t)b * P->nq + (kvh * rep + mr) * hd + 4u * mc) = o;
      }
      bar_sync(1, kConsumers);  // the merge's scratch is reused by the next item
    }
  }
  if (X.tid == kLeaderTid) PS_TRACE_PHASE(X, p, 3);
}

// ---- logits out, greedy pick ------------------------------------------------------------------------------

template <int MT>
__device__ void final_phase(Ctx<MT>& X, const PhaseDesc& D, uint32_t p) {
  const StepParams* P = X.c.sp;
  if (X.tid == kLeaderTid) grid_barrier<MT>(X, p, true);
  bar_sync(1, kConsumers);
  phase_duties<MT>(X, D);
  float rsv[MT];
  warp_rstd<MT>(X, D, rsv);
  const int ct = X.tid - kWarpLeader * 32, cw = X.warp - kWarpLeader;
  const uint32_t n = P->Vl;
  const uint32_t a = (uint32_t)((uint64_t)n * blockIdx.x / gridDim.x), b = (uint32_t)((uint64_t)n * (blockIdx.x + 1) / gridDim.x);
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    if ((uint32_t)r >= X.c.m) break;
    const float rs = rsv[r];
    const bool poisoned = __ldcg(D.poison_in + r) != 0;
    int32_t bv = INT32_MIN, bj = -1;
    for (uint32_t j = a + ct; j < b; j += kConsumers) {
      float v = unfix(__ldcg(D.acc_in + (size_t)r * n + j)) * rs;
      if (poisoned) v = __int_as_float(0x7fc00000);
      P->logits[(size_t)r * n + j] = v;
      const int32_t ov = ordered_bits(v);
      if (ov >= bv) { bv = ov; bj = (int32_t)(j + P->col_offset); }  // ascending j: >= keeps the last maximum (generation.rs:6-8)
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const int32_t ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off), oj = __shfl_xor_sync(0xFFFFFFFFu, bj, off);
      if (ov > bv || (ov == bv && oj > bj)) { bv = ov; bj = oj; }
    }
    if (X.lane == 0) X.sh->arg[r][cw] = make_int2(bv, bj);
  }
  bar_sync(1, kConsumers);
  if (ct < (int)X.c.m) {
    int2 best = X.sh->arg[ct][0];
    for (int w = 1; w < kConvWarps; ++w) {
      const int2 o = X.sh->arg[ct][w];
      if (o.x > best.x || (o.x == best.x && o.y > best.y)) best = o;
    }
    P->arg_slots[(size_t)blockIdx.x * kMaxRows + ct] = best;
  }
}

template <int MT>
__device__ void pick_phase(Ctx<MT>& X, uint32_t p) {
  const StepParams* P = X.c.sp;
  if (X.tid == kLeaderTid) grid_barrier<MT>(X, p, blockIdx.x == 0);
  bar_sync(1, kConsumers);
  if (blockIdx.x != 0 || X.aborted()) return;
  const int cw = X.warp - kWarpLeader;
  if (cw < (int)X.c.m && P->want_argmax) {
    int32_t bv = INT32_MIN, bj = -1;
    for (uint32_t t = X.lane; t < gridDim.x; t += 32) {
      const int2 o = __ldcg(P->arg_slots + (size_t)t * kMaxRows + cw);
      if (o.y >= 0 && (o.x > bv || (o.x == bv && o.y > bj))) { bv = o.x; bj = o.y; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const int32_t ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off), oj = __shfl_xor_sync(0xFFFFFFFFu, bj, off);
      if (oj >= 0 && (bj < 0 || ov > bv || (ov == bv && oj > bj))) { bv = ov; bj = oj; }
    }
    if (X.lane == 0) P->ids[cw] = bj;
  }
  if (X.tid == kLeaderTid) *P->len += 1;
}

// f32 out of the accumulator, which is left zero (test program).
template <int MT>
__device__ void out_phase(Ctx<MT>& X, const PhaseDesc& D, uint32_t p) {
  if (X.tid == kLeaderTid) grid_barrier<MT>(X, p, true);
  bar_sync(1, kConsumers);
  const int ct = X.tid - kWarpLeader * 32;
  const uint32_t total = X.c.m * D.n;
  const uint32_t a = (uint32_t)((uint64_t)total * blockIdx.x / gridDim.x), b = (uint32_t)((uint64_t)total * (blockIdx.x + 1) / gridDim.x);
  for (uint32_t i = a + ct; i < b; i += kConsumers) {
    float v = unfix(__ldcg(D.acc_in + i));
    if (__ldcg(D.poison_in + i / D.n)) v = __int_as_float(0x7fc00000);
    X.c.out[i] = v;
    const_cast<long long*>(D.acc_in)[i] = 0;
  }
}

template <int MT, typename Prog>
__device__ void run_program(const Prog& prog, unsigned char* smem, Shared* sh, uint32_t len) {
  Ctx<MT> X(smem, sh);
  X.tid = threadIdx.x; X.lane = X.tid & 31; X.warp = X.tid >> 5;
  X.s = 0; X.mc0 = 0; X.mc1 = 0; X.mc2 = 0; X.sgc = 0; X.cur_phase = 0;
  if (X.tid == 0) {
    for (int i = 0; i < kSlots; ++i) { mbar_init(&sh->b.full[i], 1); mbar_init(&sh->b.empty[i], 4); }
    for (int i = 0; i < kGroups; ++i) { mbar_init(&sh->b.a_ready[i][0], 4); mbar_init(&sh->b.a_ready[i][1], 4); mbar_init(&sh->b.mma_done[i][0], 1); mbar_init(&sh->b.mma_done[i][1], 1); }
    for (int i = 0; i < 2; ++i) {
      for (int j = 0; j < 2; ++j) { mbar_init(&sh->b.seg_done[i][j], 2); mbar_init(&sh->b.seg_free[i][j], 4); }
      mbar_init(&sh->b.fin[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    sh->abort = 0;
  }
  __syncwarp();
  if (X.warp == kWarpLeader) tmem_alloc(&sh->tmem, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  X.tmem = sh->tmem;

  const uint32_t np = prog.nphases();
  if (X.warp == 0) {
    if (X.lane == 0) {
      producer_loop<MT>(X, prog, len);
      // no copy may be in flight when the CTA leaves
      const uint32_t issued = X.s;
      for (uint32_t i = issued > (uint32_t)kSlots ? issued - kSlots : 0u; i < issued; ++i) {
        // bounded like every wait, but not cut short by the abort flag: the point is to outlast the copies
        const uint32_t a = smem_u32(&sh->b.full[i % kSlots]), parity = (i / kSlots) & 1u;
        for (unsigned poll = 0; poll < X.c.spin_limit; ++poll) {
          uint32_t ok;
          asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                       : "=r"(ok) : "r"(a), "r"(parity) : "memory");
          if (ok) break;
          __nanosleep(100);
        }
      }
    }
  } else {
    const bool scribe = X.warp == kWarpIssuer1 && X.lane == 1;  // a lane with no role of its own writes the descriptors
    if (scribe) prog.get(0, sh->D[0]);
    bar_sync(1, kConsumers);
    for (uint32_t p = 0; p < np; ++p) {
      // Between the phases: every warp of this CTA is done with phase p - 1 (the leader then joins the grid barrier
      // inside the phase), and the descriptor of phase p, written during phase p - 1, is visible.  Phase p + 1's goes
      // into a slot nobody reads any more, while the grid barrier is waited for.
      if (p > 0) bar_sync(1, kConsumers);
      if (scribe && p + 1 < np) prog.get(p + 1, sh->D[(p + 1) % 3u]);
      const PhaseDesc& D = sh->D[p % 3u];
      switch (D.type) {
        case PH_GEMV: gemv_phase<MT>(X, D, p); break;
        case PH_ATTN: attn_phase<MT>(X, D, p, len); break;
        case PH_FINAL: final_phase<MT>(X, D, p); break;
        case PH_PICK: pick_phase<MT>(X, p); break;
        default: out_phase<MT>(X, D, p); break;
      }
    }
    // every MMA has completed before the tensor memory goes back (normally their sums were all read long ago; a CTA
    // that gave up may still have some in flight)
    if ((X.warp == kWarpLeader || X.warp == kWarpIssuer1) && X.lane == 0) {
      const int ii = X.warp == kWarpLeader ? 0 : 1;
      umma_commit(&sh->b.fin[ii]);
      mbar_wait(&sh->b.fin[ii], 0);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (X.warp == kWarpLeader) tmem_dealloc(X.tmem, kTmemCols);
}

// The parameter block is copied into shared memory once and used from there; nothing takes the address of the
// kernel parameter itself.
template <int MT>
__global__ void __launch_bounds__(kThreads, 1) pstep_kernel(const StepParams Pin) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Shared sh;
  __shared__ StepParams P;
  if (threadIdx.x == 0) P = Pin;
  __syncthreads();
  LayerPtrs* lay = reinterpret_cast<LayerPtrs*>(smem + kOffLayers);
  for (uint32_t i = threadIdx.x; i < P.L * (sizeof(LayerPtrs) / 8); i += kThreads)
    reinterpret_cast<unsigned long long*>(lay)[i] = reinterpret_cast<const unsigned long long*>(P.layers)[i];
  const uint32_t len = (uint32_t)*P.len;
  __syncthreads();
  if (threadIdx.x == 0) {
    Common& cm = sh.c;
    cm.m = P.m; cm.bar = P.bar; cm.bar_base = P.bar_base; cm.status = P.status; cm.abort_flag = P.abort_flag; cm.spin_limit = P.spin_limit; cm.tx_shortfall = P.tx_shortfall;
    cm.sp = &P; cm.out = nullptr; cm.trace = P.trace;
  }
  StepProgram prog{P, lay};
  run_program<MT>(prog, smem, &sh, len);
}

template <int MT>
__global__ void __launch_bounds__(kThreads, 1) pgemv_kernel(const GemvTestParams Pin) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Shared sh;
  __shared__ GemvTestParams P;
  if (threadIdx.x == 0) P = Pin;
  __syncthreads();
  if (threadIdx.x == 0) {
    Common& cm = sh.c;
    cm.m = P.m; cm.bar = P.bar; cm.bar_base = P.bar_base; cm.status = P.status; cm.abort_flag = P.abort_flag; cm.spin_limit = P.spin_limit; cm.tx_shortfall = P.tx_shortfall;
    cm.sp = nullptr; cm.out = P.out; cm.trace = P.trace;
  }
  TestProgram prog{P};
  run_program<MT>(prog, smem, &sh, 0u);
}

template <typename K>
int launch_coop(ruai_ctx* c, K kernel, int grid, size_t smem, void* params) {
  static bool attr_done[64][4] = {};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  (void)attr_done;
  void* args[1] = {params};
  c->launches++;
  cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)kernel, args);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "persistent kernel launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}

size_t smem_bytes(uint32_t L) { return kOffLayers + (size_t)L * sizeof(LayerPtrs) + 64; }

}  // namespace ps

int ruai_pstep_grid(ruai_ctx* c) {
  static int cached[64] = {};
  int& g = cached[c->ordinal & 63];
  if (g) return g > 0 ? g : 0;
  g = -1;
  const size_t smem = ps::smem_bytes(ps::kMaxLayers);
  for (auto k : {(const void*)ps::pstep_kernel<1>, (const void*)ps::pstep_kernel<2>, (const void*)ps::pgemv_kernel<1>, (const void*)ps::pgemv_kernel<2>}) {
    const cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      ruai_fail(c, RUAI_ERR_UNSUPPORTED, "persistent kernel: %zu bytes of dynamic shared memory refused (%s)", smem, cudaGetErrorString(e));
      return 0;
    }
  }
  int per_sm = 0;
  const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ps::pstep_kernel<2>, ps::kThreads, smem);
  if (e != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    ruai_fail(c, RUAI_ERR_UNSUPPORTED, "persistent kernel: occupancy %d with %d threads and %zu bytes of shared memory (%s)", per_sm, ps::kThreads, smem,
              cudaGetErrorString(e));
    return 0;
  }
  int coop = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, c->ordinal);
  if (!coop) { ruai_fail(c, RUAI_ERR_UNSUPPORTED, "persistent kernel: the device has no cooperative launch"); return 0; }
  g = c->sm_count;
  return g;
}

int ruai_pstep_launch(ruai_ctx* c, const ps::StepParams& p) {
  const int grid = ruai_pstep_grid(c);
  if (grid <= 0) return RUAI_ERR_UNSUPPORTED;  // the reason is in the context's error text
  if (p.L > (uint32_t)ps::kMaxLayers) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "the persistent decode kernel takes at most %d layers", ps::kMaxLayers);
  ps::StepParams q = p;
  return p.m <= 1 ? ps::launch_coop(c, ps::pstep_kernel<1>, grid, ps::smem_bytes(p.L), &q)
                  : ps::launch_coop(c, ps::pstep_kernel<2>, grid, ps::smem_bytes(p.L), &q);
}

int ruai_pgemv_launch(ruai_ctx* c, const ps::GemvTestParams& p) {
  const int grid = ruai_pstep_grid(c);
  if (grid <= 0) return RUAI_ERR_UNSUPPORTED;
  ps::GemvTestParams q = p;
  return p.m <= 1 ? ps::launch_coop(c, ps::pgemv_kernel<1>, grid, ps::smem_bytes(0), &q)
                  : ps::launch_coop(c, ps::pgemv_kernel<2>, grid, ps::smem_bytes(0), &q);
}

// ---- one Linear through the persistent kernel's data path -----------------------------------------------

RUAI_API int ruai_matmul_q_stream(ruai_ctx* c, const float* x_dev, const ruai_qweight* w_in, float* out_dev, uint32_t m, uint32_t repeat) {
  if (!c || !x_dev || !w_in || !out_dev) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q_stream: NULL argument");
  if (m < 1 || m > (uint32_t)ps::kMaxRows) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_matmul_q_stream takes 1..%d rows, got %u", ps::kMaxRows, m);
  if (repeat < 1) repeat = 1;
  ruai_qweight* w = const_cast<ruai_qweight*>(w_in);
  if (!ruai_sweight_supported(w)) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_matmul_q_stream takes int8 or int4 group-32 weights with k a multiple of 4");
  DeviceGuard g(c->ordinal);
  const int grid = ruai_pstep_grid(c);
  if (grid <= 0) return RUAI_ERR_UNSUPPORTED;  // the reason is in the context's error text
  if (!w->stream) {
    w->stream = new ruai_sweight();
    const int rc = ruai_sweight_create(c, w, w->stream);
    if (rc != RUAI_OK) { delete w->stream; w->stream = nullptr; return rc; }
  }
  if (!c->ps_sync) {
    RUAI_CUDA(c, cudaMalloc(&c->ps_sync, 64));
    RUAI_CUDA(c, cudaMemsetAsync(c->ps_sync, 0, 64, c->stream));
    c->ps_bar_base = 0;
  }
  const size_t acc_bytes = (size_t)m * w->n * sizeof(long long);
  RUAI_TRY(ruai_ctx_reserve(c, acc_bytes, 0));
  RUAI_CUDA(c, cudaMemsetAsync(c->partial, 0, acc_bytes, c->stream));
  RUAI_CUDA(c, cudaMemsetAsync(c->ps_sync + 2, 0, 2 * sizeof(unsigned), c->stream));
  ps::GemvTestParams P{};
  P.m = m; P.repeat = repeat;
  P.g = ps::Geom{w->stream->ntiles, w->stream->nblk, w->stream->n, w->stream->k};
  P.bits = w->bits; P.w = w->stream->data; P.colscale = w->stream->colscale;
  P.x = x_dev; P.acc = reinterpret_cast<long long*>(c->partial); P.poison = reinterpret_cast<int*>(c->ps_sync + 2); P.out = out_dev;
  P.bar = c->ps_sync; P.bar_base = c->ps_bar_base + c->barrier_skew * (unsigned)grid; P.status = c->status;
  P.abort_flag = reinterpret_cast<int*>(c->ps_sync + 1); P.spin_limit = c->spin_limit;
  P.tx_shortfall = c->tx_shortfall;
  P.trace = c->trace;
  c->barrier_skew = 0;
  c->tx_shortfall = 0;
  RUAI_TRY(ruai_pgemv_launch(c, P));
  c->ps_bar_base += (2u * repeat - 1u) * (unsigned)grid;
  return RUAI_OK;
}

RUAI_API int ruai_ctx_set_wait_limit(ruai_ctx* c, unsigned polls) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  c->spin_limit = polls ? polls : (1u << 20);
  return RUAI_OK;
}

RUAI_API int ruai_ctx_inject_copy_shortfall(ruai_ctx* c, unsigned bytes) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  c->tx_shortfall = bytes;
  return RUAI_OK;
}

RUAI_API int ruai_ctx_inject_barrier_skew(ruai_ctx* c, unsigned grids) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  c->barrier_skew = grids;
  return RUAI_OK;
}
