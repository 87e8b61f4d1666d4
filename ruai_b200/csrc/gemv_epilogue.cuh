// The epilogue shared by the staged GEMV kernels: int8 column scale, bias, GELU / SwiGLU,
// residual add, output cast, per-tile sum of squares, per-tile argmax with the final pick.
// One thread per column; COLS threads per CTA; every thread of the CTA must call it.
#pragma once
#include "common.cuh"

__device__ __forceinline__ float gelu_ref(float x) {  // cpu.rs:229-239: 1 - 2/(exp(2u)+1), u clamped to +-15
  float u = 0.7978846f * (x + 0.044715f * x * x * x);
  u = fminf(fmaxf(u, -15.0f), 15.0f);
  const float t = 1.0f - 2.0f / (expf(2.0f * u) + 1.0f);
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ float silu_ref(float v) { return v * (1.0f / (1.0f + expf(-v))); }  // ops.rs:158-160
__device__ __forceinline__ int32_t ordered_bits(float v) {  // total_cmp order as a signed integer
  int32_t i = __float_as_int(v);
  return i ^ (int32_t)(((uint32_t)(i >> 31)) >> 1);
}

template <int MT, int COLS>
__device__ __forceinline__ void gemv_epilogue(const GemvEpilogue& e, float (&acc)[MT], uint32_t rows, uint32_t m0, uint32_t m, uint32_t j, bool active,
                                              bool scale_cols, float col_scale, void* out, float* s_red, int2* s_arg, unsigned* s_flag,
                                              const float* resid_pre = nullptr) {
  const int tid = threadIdx.x;
  const float bias = (e.bias && active) ? e.bias[j] : 0.0f;
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    if (r >= (int)rows) break;  // uniform across the CTA
    float v = acc[r];
    if (scale_cols) v *= col_scale;
    if (e.bias) v += bias;
    const size_t row = (size_t)(m0 + r);
    if (e.act == ACT_SWIGLU) {
      // columns (2i, 2i+1) hold (gate_i, up_i): layers.rs:573-576
      const float other = __shfl_xor_sync(0xFFFFFFFFu, v, 1);
      if (active && (j & 1u) == 0) {
        const float h = silu_ref(v) * other;
        const size_t o = row * e.out_ld + (j >> 1);
        store_from_f32(out, e.out_dtype, o, e.resid ? e.resid[o] + h : h);
      }
      continue;
    }
    if (active) {
      if (e.act == ACT_GELU) v = gelu_ref(v);
      const size_t o = row * e.out_ld + j;
      if (e.resid) v = (resid_pre ? resid_pre[r] : e.resid[o]) + v;  // resid_pre: the same values, fetched early
      store_from_f32(out, e.out_dtype, o, v);
    }
    if (e.sumsq) {  // sum of squares of this tile's part of the stored row, in a fixed order
      float q = active ? v * v : 0.0f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) q += __shfl_xor_sync(0xFFFFFFFFu, q, off);
      __syncthreads();
      if (lane == 0) s_red[warp] = q;
      __syncthreads();
      if (tid == 0) {
        float t = 0.0f;
        for (int w = 0; w < COLS / 32; ++w) t += s_red[w];
        e.sumsq[(size_t)blockIdx.x * m + row] = t;
      }
    }
    if (e.argmax_out) {  // best (value, column) of this tile; ties go to the larger column
      int32_t bv = active ? ordered_bits(v) : INT32_MIN;
      int32_t bj = active ? (int32_t)j : -1;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const int32_t ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
        const int32_t oj = __shfl_xor_sync(0xFFFFFFFFu, bj, off);
        if (ov > bv || (ov == bv && oj > bj)) { bv = ov; bj = oj; }
      }
      __syncthreads();
      if (lane == 0) s_arg[warp] = make_int2(bv, bj);
      __syncthreads();
      if (tid == 0) {
        int2 b = s_arg[0];
        for (int w = 1; w < COLS / 32; ++w)
          if (s_arg[w].x > b.x || (s_arg[w].x == b.x && s_arg[w].y > b.y)) b = s_arg[w];
        e.argmax_slots[(size_t)blockIdx.x * m + row] = b;
      }
    }
  }
  if (e.argmax_out) {
    // the last column tile to finish picks the winners and advances the position
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned a = atomicAdd(e.argmax_counter, 1u);
      *s_flag = a == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (*s_flag) {
      __threadfence();
      // one warp per row: the lanes share the tiles, then the best of the 32 by shuffles
      const volatile int* sl = (const volatile int*)e.argmax_slots;
      for (uint32_t row = warp; row < m; row += COLS / 32) {
        int bv = INT32_MIN, bj = -1;
        for (uint32_t t = lane; t < gridDim.x; t += 32) {
          const int v = sl[2 * ((size_t)t * m + row)], jj = sl[2 * ((size_t)t * m + row) + 1];
          if (v > bv || (v == bv && jj > bj)) { bv = v; bj = jj; }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const int ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
          const int oj = __shfl_xor_sync(0xFFFFFFFFu, bj, off);
          if (ov > bv || (ov == bv && oj > bj)) { bv = ov; bj = oj; }
        }
        if (lane == 0) e.argmax_out[row] = bj;
      }
      if (tid == 0) {
        *e.argmax_counter = 0;
        if (e.len_ptr) *e.len_ptr += e.len_add;
      }
    }
  }
}
