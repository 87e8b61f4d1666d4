// One-shot push all-reduce and vocabulary-parallel argmax over NVLink peer memory.
//
// The reference has no distributed layer at all; this is the exchange step that
// Megatron-style sharding of the Linear weights adds: one sum of [rows, d] f32 after the
// attention output projection and one after the MLP down projection.  At decode sizes
// (16 KB per exchange) a library all-reduce is latency bound, so each rank stores its
// partial sums straight into a receive slot in every peer's memory, raises a flag
// there, waits for the peers' flags in its own memory and adds the slots in rank order,
// which gives every rank bit-identical results.  Slots and flags are double buffered by
// the parity of a sequence number kept on the device (so the kernels can sit in a
// replayed graph).  Every wait is bounded: on a timeout the kernel records status 2 and
// returns.  Only plain peer loads and stores are used.
#include "tp.cuh"

namespace {


struct TpDev {
  uint32_t rank, world;
  size_t slot_floats;
  unsigned* flags[kTpMaxWorld];   // per rank: [2][world][kTpMaxCtas]
  unsigned* aflags[kTpMaxWorld];  // per rank: [2][world][kTpArgmaxRows]
  int2* aslots[kTpMaxWorld];      // per rank: [2][world][kTpArgmaxRows]
  float* data[kTpMaxWorld];       // per rank: [2][world][slot_floats]
  unsigned* seq;
  unsigned spin_limit;            // polls (about 100 ns apart) a wait for a peer may take: by default about half a second
};

size_t flags_bytes() { return 2ull * kTpMaxWorld * kTpMaxCtas * sizeof(unsigned); }
size_t aflags_bytes() { return 2ull * kTpMaxWorld * kTpArgmaxRows * sizeof(unsigned); }
size_t aslots_bytes() { return 2ull * kTpMaxWorld * kTpArgmaxRows * sizeof(int2); }

TpDev make_dev(const ruai_ctx* c, const ruai_tp_state* t) {
  TpDev d;
  d.rank = t->rank; d.world = t->world; d.slot_floats = t->slot_floats; d.seq = t->seq;
  d.spin_limit = c->spin_limit < (1u << 30) ? c->spin_limit << 2 : 0xFFFFFFFFu;  // ruai_ctx_set_wait_limit scales both kinds of waits
  for (uint32_t p = 0; p < kTpMaxWorld; ++p) {
    char* base = (char*)t->peer[p];
    d.flags[p] = (unsigned*)base;
    d.aflags[p] = base ? (unsigned*)(base + flags_bytes()) : nullptr;
    d.aslots[p] = base ? (int2*)(base + flags_bytes() + aflags_bytes()) : nullptr;
    d.data[p] = base ? (float*)(base + flags_bytes() + aflags_bytes() + aslots_bytes()) : nullptr;
  }
  return d;
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Returns false when the flag did not reach `want` within the limit.
__device__ bool bounded_wait(const unsigned* flag, unsigned want, unsigned limit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (ld_acquire_sys(flag) == want) return true;
    __nanosleep(100);
  }
  return false;
}

__global__ void __launch_bounds__(256) allreduce_push_kernel(TpDev t, const float* __restrict__ partial, float* __restrict__ x, uint32_t count4,
                                                             int* err, float* __restrict__ sumsq) {
  __shared__ int s_ok;
  __shared__ float s_sq[8];
  grid_dependency_wait();
  grid_launch_dependents();
  const unsigned seq = *(volatile unsigned*)&t.seq[0] + 1u;
  const unsigned par = seq & 1u;
  const uint32_t per = (count4 + gridDim.x - 1) / gridDim.x;
  const uint32_t i0 = blockIdx.x * per, i1 = min(count4, i0 + per);
  const float4* src = reinterpret_cast<const float4*>(partial);
  // push this rank's share of the partial sums into every peer's slot
  for (uint32_t p = 0; p < t.world; ++p) {
    if (p == t.rank) continue;
    float4* dst = reinterpret_cast<float4*>(t.data[p] + ((size_t)par * t.world + t.rank) * t.slot_floats);
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) dst[i] = src[i];
  }
  __threadfence_system();
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < t.world && threadIdx.x != t.rank)
    st_release_sys(&t.flags[threadIdx.x][((size_t)par * t.world + t.rank) * kTpMaxCtas + blockIdx.x], seq);
  if (threadIdx.x < t.world && threadIdx.x != t.rank) {
    if (!bounded_wait(&t.flags[t.rank][((size_t)par * t.world + threadIdx.x) * kTpMaxCtas + blockIdx.x], seq, t.spin_limit)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) atomicExch(err, 2);
  } else {
    float4* xv = reinterpret_cast<float4*>(x);
    float sq = 0.0f;
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (uint32_t p = 0; p < t.world; ++p) {  // rank order: identical bits everywhere
        const float4 v = p == t.rank ? src[i]
                                     : __ldcv(reinterpret_cast<const float4*>(t.data[t.rank] + ((size_t)par * t.world + p) * t.slot_floats) + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      float4 r = xv[i];
      r.x += s.x; r.y += s.y; r.z += s.z; r.w += s.w;
      xv[i] = r;
      sq = fmaf(r.x, r.x, sq); sq = fmaf(r.y, r.y, sq); sq = fmaf(r.z, r.z, sq); sq = fmaf(r.w, r.w, sq);
    }
    if (sumsq) {  // single-CTA, single-row launches only: the sum of squares the next RMSNorm needs, in a fixed order
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
      if ((threadIdx.x & 31) == 0) s_sq[threadIdx.x >> 5] = sq;
      __syncthreads();
      if (threadIdx.x == 0) {
        float tot = 0.0f;
        for (int w = 0; w < 8; ++w) tot += s_sq[w];
        sumsq[0] = tot;
      }
    }
  }
  // the last CTA to finish advances the sequence number
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned a = atomicAdd(&t.seq[2], 1u);
    if (a == gridDim.x - 1) {
      t.seq[2] = 0;
      __threadfence();
      *(volatile unsigned*)&t.seq[0] = seq;
    }
  }
}

__device__ __forceinline__ int32_t total_order(float v) {
  int32_t i = __float_as_int(v);
  return i ^ (int32_t)(((uint32_t)(i >> 31)) >> 1);
}

// One CTA per row: local argmax (last maximum), exchange of (value, global index), global pick.
__global__ void __launch_bounds__(1024) tp_argmax_kernel(TpDev t, const float* __restrict__ logits, uint32_t n, uint32_t col_offset,
                                                         int32_t* __restrict__ out, int* err) {
  __shared__ int32_t sv[32];
  __shared__ uint32_t si[32];
  __shared__ int s_ok;
  grid_dependency_wait();
  grid_launch_dependents();
  const unsigned seq = *(volatile unsigned*)&t.seq[1] + 1u;
  const unsigned par = seq & 1u;
  const uint32_t row = blockIdx.x;
  const float* lr = logits + (size_t)row * n;
  int32_t bv = INT32_MIN;
  uint32_t bi = 0;
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
    const int32_t v = total_order(lr[i]);
    if (v >= bv) { bv = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const int32_t ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
    if (ov > bv || (ov == bv && oi > bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { sv[w] = bv; si[w] = bi; }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < nw; ++i)
      if (sv[i] > sv[0] || (sv[i] == sv[0] && si[i] > si[0])) { sv[0] = sv[i]; si[0] = si[i]; }
    si[0] += col_offset;
  }
  __syncthreads();
  const int2 mine = make_int2(sv[0], (int)si[0]);
  if (threadIdx.x < t.world && threadIdx.x != t.rank) {
    const size_t slot = ((size_t)par * t.world + t.rank) * kTpArgmaxRows + row;
    t.aslots[threadIdx.x][slot] = mine;
    __threadfence_system();
    st_release_sys(&t.aflags[threadIdx.x][slot], seq);
    const size_t theirs = ((size_t)par * t.world + threadIdx.x) * kTpArgmaxRows + row;
    if (!bounded_wait(&t.aflags[t.rank][theirs], seq, t.spin_limit)) s_ok = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!s_ok) atomicExch(err, 2);
    else {
      int2 best = mine;
      for (uint32_t p = 0; p < t.world; ++p) {
        if (p == t.rank) continue;
        const volatile int* vp = (const volatile int*)&t.aslots[t.rank][((size_t)par * t.world + p) * kTpArgmaxRows + row];
        const int2 v = make_int2(vp[0], vp[1]);
        if (v.x > best.x || (v.x == best.x && v.y > best.y)) best = v;
      }
      out[row] = best.y;
    }
    __threadfence();
    const unsigned a = atomicAdd(&t.seq[3], 1u);
    if (a == gridDim.x - 1) {
      t.seq[3] = 0;
      __threadfence();
      *(volatile unsigned*)&t.seq[1] = seq;
    }
  }
}

}  // namespace

int ruai_tp_init(ruai_ctx* c, ruai_tp_state* t, uint32_t rank, uint32_t world, uint32_t d) {
  if (world > kTpMaxWorld) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "tensor-parallel world %u > %u", world, kTpMaxWorld);
  t->rank = rank; t->world = world;
  const uint32_t slot_rows = 1024;
  t->slot_floats = (size_t)slot_rows * d;
  t->region_bytes = flags_bytes() + aflags_bytes() + aslots_bytes() + 2ull * world * t->slot_floats * sizeof(float);
  RUAI_CUDA(c, cudaMalloc(&t->region, t->region_bytes));
  RUAI_CUDA(c, cudaMemset(t->region, 0, flags_bytes() + aflags_bytes() + aslots_bytes()));
  RUAI_CUDA(c, cudaMalloc(&t->partial, t->slot_floats * sizeof(float)));
  RUAI_CUDA(c, cudaMalloc(&t->seq, 4 * sizeof(unsigned)));
  RUAI_CUDA(c, cudaMemset(t->seq, 0, 4 * sizeof(unsigned)));
  t->peer[rank] = t->region;
  return RUAI_OK;
}

void ruai_tp_destroy(ruai_tp_state* t) {
  for (uint32_t p = 0; p < kTpMaxWorld; ++p)
    if (t->peer[p] && p != t->rank) cudaIpcCloseMemHandle(t->peer[p]);
  if (t->region) cudaFree(t->region);
  if (t->partial) cudaFree(t->partial);
  if (t->seq) cudaFree(t->seq);
  *t = ruai_tp_state();
}

// After an exchange that timed out the ranks' sequence numbers no longer agree.  Every rank, with none of its kernels in
// flight and after all ranks have stopped stepping (the caller's barrier), clears its own flags and counts; after a
// second barrier of the caller's the exchange starts again from sequence 0.
int ruai_tp_resync_state(ruai_ctx* c, ruai_tp_state* t) {
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  RUAI_CUDA(c, cudaMemset(t->region, 0, flags_bytes() + aflags_bytes() + aslots_bytes()));
  RUAI_CUDA(c, cudaMemset(t->seq, 0, 4 * sizeof(unsigned)));
  RUAI_CUDA(c, cudaDeviceSynchronize());
  return RUAI_OK;
}

int ruai_tp_export_handle(ruai_ctx* c, ruai_tp_state* t, void* handle_out) {
  static_assert(sizeof(cudaIpcMemHandle_t) == RUAI_IPC_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  RUAI_CUDA(c, cudaIpcGetMemHandle(&h, t->region));
  memcpy(handle_out, &h, sizeof h);
  return RUAI_OK;
}

int ruai_tp_connect_handles(ruai_ctx* c, ruai_tp_state* t, const void* handles) {
  for (uint32_t p = 0; p < t->world; ++p) {
    if (p == t->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char*)handles + (size_t)p * RUAI_IPC_HANDLE_BYTES, sizeof h);
    RUAI_CUDA(c, cudaIpcOpenMemHandle(&t->peer[p], h, cudaIpcMemLazyEnablePeerAccess));
  }
  t->connected = true;
  return RUAI_OK;
}

int ruai_tp_check_ready(ruai_ctx* c, ruai_tp_state* t, uint32_t rows, uint32_t d) {
  if (!t->connected) return ruai_fail(c, RUAI_ERR_COMM, "tensor-parallel ranks are not connected: exchange ruai_tp_export handles and call ruai_tp_connect");
  if ((size_t)rows * d > t->slot_floats) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "%u rows exceed the exchange slot (%zu rows)", rows, t->slot_floats / d);
  if (d % 4) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "hidden size %u must be a multiple of 4 for the exchange", d);
  return RUAI_OK;
}

bool ruai_tp_allreduce_gives_sumsq(uint32_t rows, uint32_t d) { return rows == 1 && d / 4 <= 1024; }

int ruai_tp_allreduce_add(ruai_ctx* c, ruai_tp_state* t, float* x, uint32_t rows, uint32_t d, int* err, float* sumsq) {
  const uint32_t count4 = (uint32_t)((size_t)rows * d / 4);
  uint32_t ctas = (count4 + 1023) / 1024;  // 4 float4 per thread
  ctas = ctas < 1 ? 1 : (ctas > kTpMaxCtas ? kTpMaxCtas : ctas);
  if (sumsq && !(ctas == 1 && rows == 1)) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "the exchange gives the sum of squares only for one row in one CTA");
  RUAI_CUDA(c, ruai_launch(c, allreduce_push_kernel, dim3(ctas), dim3(256), 0, true, make_dev(c, t), (const float*)t->partial, x, count4, err, sumsq));
  return RUAI_OK;
}

int ruai_tp_argmax(ruai_ctx* c, ruai_tp_state* t, const float* logits, uint32_t n_local, uint32_t rows, uint32_t col_offset, int32_t* out, int* err) {
  if (rows > kTpArgmaxRows) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "argmax over %u rows exceeds %u", rows, kTpArgmaxRows);
  RUAI_CUDA(c, ruai_launch(c, tp_argmax_kernel, dim3(rows), dim3(1024), 0, true, make_dev(c, t), logits, n_local, col_offset, out, err));
  return RUAI_OK;
}
