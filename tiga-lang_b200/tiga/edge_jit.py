"""Runtime-compiled edge programs: CUDA source for ONE staged edge expression.

``tiga.edge_program`` compiles an ``edge()`` expression to a register program that the kernels of
``csrc/tgb_edge_program.cu`` interpret.  This module writes the same three passes (forward fold,
destination-major and source-major reverse mode, each with its one-CTA-per-long-row companion) as
CUDA source in which the program is straight-line code -- one line per instruction for the
evaluation, one per instruction for the reverse sweep, operand roles and widths as compile-time
tables -- and has the library compile it for sm_100a with NVRTC (``tgb_jit_build``).  The
arithmetic, the order of every sum and the launch geometry are those of the interpreter, so the two
give the same bits; what changes is the instruction count per edge (the interpreter spends about
ten instructions and a trip through local memory per program instruction).

This is what the reference's provider pipeline does with a captured UDF: generated kernel code,
compiled at run time and cached per specialisation (python/tiga/codegen/ttir.py:103-121 and
python/tiga/interop/torch/message_passing.py:2579-2815 of walkerchi/TIGA-lang; its generator emits
TTIR for Triton).  Modules are cached per (program structure, reducer, message width, operand
moduli); parameter-fed constants are launch arguments, not part of the source.
"""
from __future__ import annotations

import ctypes
import os
import sys
import threading

from . import _native
from . import edge_program as ep

_PRELUDE = r"""
typedef long long i64;
typedef int i32;
typedef unsigned int u32;

struct Args {
  const float *in[8];
  float *sink[8];
  const void *ptr;
  const void *idx;
  const u32 *eid;
  const i32 *order;
  const void *degree_ptr;
  const float *dy;
  float *out;
  float *saved_value;
  i32 *saved_index;
  i64 n_rows;
  i64 n_long;
  i64 split_threshold;
  i32 ptr_bits, idx_bits, degree_bits;
  float identity;
  float constants[16];
  const float *seeds;
  float *prefix;
  float *message_grads;
  i64 num_edges;
};

#define REDUCER_SUM 0
#define REDUCER_MEAN 1
#define REDUCER_MAX 2
#define REDUCER_PROD 3
#define REDUCER_SEEDED 4
#define ROLE_SRC 0
#define ROLE_DST 1
#define ROLE_EDGE 2
#define ROLE_PARAM 3
#define THREADS 128

__device__ __forceinline__ i64 load_index(const void *base, int bits, i64 i) {
  return bits == 64 ? __ldg(static_cast<const i64 *>(base) + i) : (i64)__ldg(static_cast<const i32 *>(base) + i);
}
__device__ __forceinline__ float quiet_nan() { return __int_as_float(0x7fc00000); }
__device__ __forceinline__ float maximum_nan(float x, float y) { return (x != x || y != y) ? quiet_nan() : fmaxf(x, y); }
__device__ __forceinline__ bool max_takes(float state, float m) { return state == state && (m != m || m > state); }
__device__ __forceinline__ unsigned group_mask() {
  return LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u) << ((threadIdx.x & 31) / LANES * LANES);
}
__device__ __forceinline__ float group_sum(float v, unsigned mask) {
#pragma unroll
  for (int offset = LANES / 2; offset > 0; offset >>= 1) v += __shfl_xor_sync(mask, v, offset, LANES);
  return v;
}
"""

_KERNELS = r"""
template <bool LONG>
__device__ __forceinline__ void forward_pass(const Args &a) {
  constexpr int kGroups = (LONG ? LONG_THREADS : THREADS) / LANES;
  __shared__ float part[LONG ? LONG_THREADS : 1];
  __shared__ float part_masked[LONG ? LONG_THREADS : 1];
  __shared__ i32 part_mark[LONG ? LONG_THREADS : 1];
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  // the plan's row order: the rows above the split threshold first (one CTA each), then the others
  // bucketed by degree, so the lane groups of a CTA walk rows of similar length
  i64 row;
  if (LONG) {
    row = __ldg(a.order + blockIdx.x);
  } else {
    const i64 position = a.n_long + (i64)blockIdx.x * kGroups + group;
    if (position >= a.n_rows) return;
    row = __ldg(a.order + position);
  }
  i64 begin = load_index(a.ptr, a.ptr_bits, row), end = load_index(a.ptr, a.ptr_bits, row + 1);
  const i64 degree = end - begin;
  if (LONG) {
    const i64 slice = (degree + kGroups - 1) / kGroups;
    begin = begin + group * slice;
    end = begin + slice < end ? begin + slice : end;
  }
  constexpr bool is_max = REDUCER == REDUCER_MAX, is_prod = REDUCER == REDUCER_PROD;
  float value[N_INSTR];
  for (int f0 = 0; f0 < WIDTH; f0 += LANES) {
    const int f = f0 + lane;
    float acc = is_max ? a.identity : is_prod ? (LONG ? 1.0f : a.identity)
                                              : ((LONG || REDUCER == REDUCER_MEAN) ? 0.0f : a.identity);
    float masked = acc;
    i32 mark = is_max ? -1 : 0;
    if (f < WIDTH) {
      for (i64 e = begin; e < end; ++e) {
        evaluate(a, load_index(a.idx, a.idx_bits, e), row, e, f, value);
        const float m = value[N_INSTR - 1];
        if (is_max) {
          if (max_takes(acc, m)) mark = (i32)e;
          acc = maximum_nan(acc, m);
        } else if (is_prod) {
          acc = __fmul_rn(acc, m);
          masked = __fmul_rn(masked, m == 0.0f ? 1.0f : m);
          mark += m == 0.0f;
        } else {
          acc = __fadd_rn(acc, m);
        }
      }
    }
    if (LONG) {
      part[group * LANES + lane] = acc;
      part_masked[group * LANES + lane] = masked;
      part_mark[group * LANES + lane] = mark;
      __syncthreads();
      if (group == 0 && f < WIDTH) {
        constexpr bool from_identity = REDUCER == REDUCER_SUM || is_prod;
        float total = from_identity ? a.identity : acc;
        float masked_total = a.identity;
        i32 mark_total = is_prod ? 0 : mark;
        for (int g = from_identity ? 0 : 1; g < kGroups; ++g) {
          const float q = part[g * LANES + lane];
          if (is_max) {
            if (max_takes(total, q)) mark_total = part_mark[g * LANES + lane];
            total = maximum_nan(total, q);
          } else if (is_prod) {
            total = __fmul_rn(total, q);
            masked_total = __fmul_rn(masked_total, part_masked[g * LANES + lane]);
            mark_total += part_mark[g * LANES + lane];
          } else {
            total = __fadd_rn(total, q);
          }
        }
        acc = total;
        masked = masked_total;
        mark = mark_total;
      }
      __syncthreads();
      if (group != 0) continue;
    }
    if (f < WIDTH) {
      if (REDUCER == REDUCER_MEAN) acc = __fdiv_rn(acc, (float)degree);
      a.out[row * WIDTH + f] = acc;
      if (a.saved_value) a.saved_value[row * WIDTH + f] = masked;
      if (a.saved_index) a.saved_index[row * WIDTH + f] = mark;
    }
  }
}

template <bool SOURCE_MAJOR, bool LONG>
__device__ __forceinline__ void reverse_pass(const Args &a) {
  constexpr int kGroups = (LONG ? LONG_THREADS : THREADS) / LANES;
  __shared__ float part_full[LONG ? N_OPERANDS * LONG_THREADS : 1];
  __shared__ float part_scalar[LONG ? N_OPERANDS * LONG_THREADS : 1];
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  i64 row;
  if (LONG) {
    row = __ldg(a.order + blockIdx.x);
  } else {
    const i64 position = a.n_long + (i64)blockIdx.x * kGroups + group;
    if (position >= a.n_rows) return;
    row = __ldg(a.order + position);
  }
  const unsigned mask = group_mask();
  i64 begin = load_index(a.ptr, a.ptr_bits, row), end = load_index(a.ptr, a.ptr_bits, row + 1);
  if (LONG) {
    const i64 slice = (end - begin + kGroups - 1) / kGroups;
    begin = begin + group * slice;
    end = begin + slice < end ? begin + slice : end;
  }
  float value[N_INSTR], adjoint[N_INSTR];
  float scalar_total[N_OPERANDS];
#pragma unroll
  for (int k = 0; k < N_OPERANDS; ++k) scalar_total[k] = 0.0f;
  constexpr int chunks = (WIDTH + LANES - 1) / LANES;
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int f = chunk * LANES + lane;
    const bool live = f < WIDTH;
    float full_total[N_OPERANDS];
#pragma unroll
    for (int k = 0; k < N_OPERANDS; ++k) full_total[k] = 0.0f;
    for (i64 t = begin; t < end; ++t) {
      const i64 other = load_index(a.idx, a.idx_bits, t);
      const i64 edge = a.eid ? (i64)__ldg(a.eid + t) : t;
      const i64 src = SOURCE_MAJOR ? row : other, dst = SOURCE_MAJOR ? other : row;
#pragma unroll
      for (int i = 0; i < N_INSTR; ++i) adjoint[i] = 0.0f;
      if (live && REDUCER == REDUCER_SEEDED) {         // message cotangents handed over per edge (user algebras)
        evaluate(a, src, dst, edge, f, value);
#pragma unroll
        for (int j = 0; j < N_MESSAGES; ++j)
          adjoint[kMessageSlot[j]] += __ldg(a.seeds + ((i64)j * a.num_edges + edge) * WIDTH + f);
        sweep_back(value, adjoint);
      } else if (live) {
        evaluate(a, src, dst, edge, f, value);
        float g = __ldg(a.dy + dst * WIDTH + f);
        if (REDUCER == REDUCER_MEAN) {
          const i64 degree = load_index(a.degree_ptr, a.degree_bits, dst + 1) - load_index(a.degree_ptr, a.degree_bits, dst);
          g = g / (float)degree;
        } else if (REDUCER == REDUCER_MAX) {
          if (__ldg(a.saved_index + dst * WIDTH + f) != (i32)edge) g = 0.0f;
        } else if (REDUCER == REDUCER_PROD) {
          const float m = value[N_INSTR - 1];
          const float others = __ldg(a.saved_value + dst * WIDTH + f);
          const i32 zeros = __ldg(a.saved_index + dst * WIDTH + f);
          g = zeros == 0 ? __fdiv_rn(__fmul_rn(g, others), m)
                         : (zeros == 1 && m == 0.0f) ? __fmul_rn(g, others) : 0.0f;
        }
        adjoint[N_INSTR - 1] = g;
        sweep_back(value, adjoint);
      }
#pragma unroll
      for (int k = 0; k < N_OPERANDS; ++k) {
        float *sink = a.sink[k];
        if (sink == nullptr) continue;
        constexpr_role_modulus(k);
        const bool full = modulus == 0 || WIDTH == 1;
        const float gk = live ? adjoint[load_slot] : 0.0f;
        if (role == ROLE_EDGE) {
          if (SOURCE_MAJOR) continue;
          if (full) {
            if (live) sink[edge * WIDTH + f] = gk;
          } else {
            const float total = group_sum(gk, mask);
            if (lane == 0) sink[edge] = chunk == 0 ? total : sink[edge] + total;
          }
        } else if ((role == ROLE_SRC) == SOURCE_MAJOR) {
          if (full) full_total[k] += gk; else scalar_total[k] += gk;
        }
      }
    }
    if (LONG) {
#pragma unroll
      for (int k = 0; k < N_OPERANDS; ++k) part_full[k * LONG_THREADS + threadIdx.x] = full_total[k];
      __syncthreads();
      if (group == 0) {
#pragma unroll
        for (int k = 0; k < N_OPERANDS; ++k) {
          float total = 0.0f;
          for (int g = 0; g < kGroups; ++g) total += part_full[k * LONG_THREADS + g * LANES + lane];
          full_total[k] = total;
        }
      }
      __syncthreads();
    }
    if (!LONG || group == 0) {
#pragma unroll
      for (int k = 0; k < N_OPERANDS; ++k) {
        constexpr_role_modulus(k);
        if (a.sink[k] == nullptr || role == ROLE_EDGE || (role == ROLE_SRC) != SOURCE_MAJOR) continue;
        const bool full = modulus == 0 || WIDTH == 1;
        if (full && live) a.sink[k][row * WIDTH + f] = full_total[k];
      }
    }
  }
  if (LONG) {
#pragma unroll
    for (int k = 0; k < N_OPERANDS; ++k) {
      const float total = group_sum(scalar_total[k], mask);
      if (lane == 0) part_scalar[k * LONG_THREADS + group] = total;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
      for (int k = 0; k < N_OPERANDS; ++k) {
        constexpr_role_modulus(k);
        if (a.sink[k] == nullptr || role == ROLE_EDGE || (role == ROLE_SRC) != SOURCE_MAJOR) continue;
        if (modulus == 0 || WIDTH == 1) continue;
        float total = 0.0f;
        for (int g = 0; g < kGroups; ++g) total += part_scalar[k * LONG_THREADS + g];
        a.sink[k][row] = total;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < N_OPERANDS; ++k) {
      constexpr_role_modulus(k);
      if (a.sink[k] == nullptr || role == ROLE_EDGE || (role == ROLE_SRC) != SOURCE_MAJOR) continue;
      if (modulus == 0 || WIDTH == 1) continue;
      const float total = group_sum(scalar_total[k], mask);
      if (lane == 0) a.sink[k][row] = total;
    }
  }
}

extern "C" __global__ void __launch_bounds__(THREADS) fwd(const __grid_constant__ Args a) { forward_pass<false>(a); }
extern "C" __global__ void __launch_bounds__(LONG_THREADS) fwd_long(const __grid_constant__ Args a) { forward_pass<true>(a); }
extern "C" __global__ void __launch_bounds__(THREADS) bwd_rows(const __grid_constant__ Args a) { reverse_pass<false, false>(a); }
extern "C" __global__ void __launch_bounds__(LONG_THREADS) bwd_rows_long(const __grid_constant__ Args a) { reverse_pass<false, true>(a); }
extern "C" __global__ void __launch_bounds__(THREADS) bwd_sources(const __grid_constant__ Args a) { reverse_pass<true, false>(a); }
extern "C" __global__ void __launch_bounds__(LONG_THREADS) bwd_sources_long(const __grid_constant__ Args a) { reverse_pass<true, true>(a); }
"""

_ALGEBRA_KERNELS = r"""
#define MAX_ARGS (ARITY + (ARITY > N_MESSAGES ? ARITY : N_MESSAGES))

__device__ __forceinline__ void fold_edge(const float *value, float *state) {
  float args[MAX_ARGS], rv[N_STEP];
#pragma unroll
  for (int k = 0; k < ARITY; ++k) args[k] = state[k];
#pragma unroll
  for (int j = 0; j < N_MESSAGES; ++j) args[ARITY + j] = value[kMessageSlot[j]];
  step_eval(args, rv);
  step_out(rv, state);
}

struct RowSpan { i64 row, begin, end, degree, slice; };

template <bool LONG>
__device__ __forceinline__ bool row_span(const Args &a, RowSpan &span) {
  constexpr int kGroups = (LONG ? LONG_THREADS : THREADS) / LANES;
  const int group = threadIdx.x / LANES;
  if (LONG) {
    span.row = __ldg(a.order + blockIdx.x);
  } else {
    const i64 position = a.n_long + (i64)blockIdx.x * kGroups + group;
    if (position >= a.n_rows) return false;
    span.row = __ldg(a.order + position);
  }
  span.begin = load_index(a.ptr, a.ptr_bits, span.row);
  span.end = load_index(a.ptr, a.ptr_bits, span.row + 1);
  span.degree = span.end - span.begin;
  span.slice = 0;
  if (LONG) {
    span.slice = (span.degree + kGroups - 1) / kGroups;
    span.begin = span.begin + group * span.slice;
    span.end = span.begin + span.slice < span.end ? span.begin + span.slice : span.end;
  }
  return true;
}

template <bool LONG>
__device__ __forceinline__ void algebra_forward(const Args &a) {
  constexpr int kGroups = (LONG ? LONG_THREADS : THREADS) / LANES;
  __shared__ float part[LONG ? ARITY * LONG_THREADS : 1];
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  RowSpan span;
  if (!row_span<LONG>(a, span)) return;
  float value[N_INSTR], state[ARITY];
  for (int f0 = 0; f0 < WIDTH; f0 += LANES) {
    const int f = f0 + lane;
    const bool live = f < WIDTH;
#pragma unroll
    for (int k = 0; k < ARITY; ++k) state[k] = identity_of(k);
    if (live) {
      for (i64 e = span.begin; e < span.end; ++e) {
        evaluate(a, load_index(a.idx, a.idx_bits, e), span.row, e, f, value);
        fold_edge(value, state);
      }
    }
    if (LONG) {
#pragma unroll
      for (int k = 0; k < ARITY; ++k) part[k * LONG_THREADS + threadIdx.x] = state[k];
      __syncthreads();
      if (group == 0 && live) {
#pragma unroll
        for (int k = 0; k < ARITY; ++k) state[k] = identity_of(k);
        for (int g = 0; g < kGroups && (i64)g * span.slice < span.degree; ++g) {
          float args[2 * ARITY], rv[N_COMBINE];
#pragma unroll
          for (int k = 0; k < ARITY; ++k) {
            args[k] = state[k];
            args[ARITY + k] = part[k * LONG_THREADS + g * LANES + lane];
          }
          combine_eval(args, rv);
          combine_out(rv, state);
        }
      }
      __syncthreads();
      if (group != 0) continue;
    }
    if (live) {
      float rv[N_FINAL], result[1];
      finalize_eval(state, rv);
      finalize_out(rv, result);
      a.out[span.row * WIDTH + f] = result[0];
    }
  }
}

template <bool LONG>
__device__ __forceinline__ void algebra_messages(const Args &a) {
  constexpr int kGroups = (LONG ? LONG_THREADS : THREADS) / LANES;
  __shared__ float part[LONG ? ARITY * LONG_THREADS : 1];
  __shared__ float joined[LONG ? ARITY * LONG_THREADS : 1];
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  RowSpan span;
  if (!row_span<LONG>(a, span)) return;
  float value[N_INSTR], state[ARITY], carried[ARITY];
  for (int f0 = 0; f0 < WIDTH; f0 += LANES) {
    const int f = f0 + lane;
    const bool live = f < WIDTH;
#pragma unroll
    for (int k = 0; k < ARITY; ++k) state[k] = identity_of(k);
    if (live) {
      for (i64 e = span.begin; e < span.end; ++e) {
#pragma unroll
        for (int k = 0; k < ARITY; ++k) a.prefix[(e * ARITY + k) * WIDTH + f] = state[k];
        evaluate(a, load_index(a.idx, a.idx_bits, e), span.row, e, f, value);
        fold_edge(value, state);
      }
    }
#pragma unroll
    for (int k = 0; k < ARITY; ++k) carried[k] = 0.0f;
    if (!LONG) {
      if (live) {
        float rv[N_FINAL], radj[N_FINAL];
        const float g = __ldg(a.dy + span.row * WIDTH + f);
        finalize_eval(state, rv);
        finalize_seed(radj, &g);
        finalize_back(rv, radj);
        finalize_args(radj, carried);
      }
    } else {
#pragma unroll
      for (int k = 0; k < ARITY; ++k) part[k * LONG_THREADS + threadIdx.x] = state[k];
      __syncthreads();
      if (group == 0 && live) {
        int used = 0;
#pragma unroll
        for (int k = 0; k < ARITY; ++k) state[k] = identity_of(k);
        for (int g = 0; g < kGroups && (i64)g * span.slice < span.degree; ++g, ++used) {
          float args[2 * ARITY], rv[N_COMBINE];
#pragma unroll
          for (int k = 0; k < ARITY; ++k) {
            joined[k * LONG_THREADS + g * LANES + lane] = state[k];
            args[k] = state[k];
            args[ARITY + k] = part[k * LONG_THREADS + g * LANES + lane];
          }
          combine_eval(args, rv);
          combine_out(rv, state);
        }
        {
          float rv[N_FINAL], radj[N_FINAL];
          const float g_row = __ldg(a.dy + span.row * WIDTH + f);
          finalize_eval(state, rv);
          finalize_seed(radj, &g_row);
          finalize_back(rv, radj);
          finalize_args(radj, carried);
        }
        for (int g = used - 1; g >= 0; --g) {
          float args[2 * ARITY], rv[N_COMBINE], radj[N_COMBINE], arg_adjoint[2 * ARITY];
#pragma unroll
          for (int k = 0; k < ARITY; ++k) {
            args[k] = joined[k * LONG_THREADS + g * LANES + lane];
            args[ARITY + k] = part[k * LONG_THREADS + g * LANES + lane];
          }
          combine_eval(args, rv);
          combine_seed(radj, carried);
          combine_back(rv, radj);
          combine_args(radj, arg_adjoint);
#pragma unroll
          for (int k = 0; k < ARITY; ++k) {
            carried[k] = arg_adjoint[k];
            part[k * LONG_THREADS + g * LANES + lane] = arg_adjoint[ARITY + k];
          }
        }
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < ARITY; ++k) carried[k] = part[k * LONG_THREADS + threadIdx.x];
    }
    if (live) {
      for (i64 e = span.end - 1; e >= span.begin; --e) {
        float args[MAX_ARGS], rv[N_STEP], radj[N_STEP], arg_adjoint[MAX_ARGS];
        evaluate(a, load_index(a.idx, a.idx_bits, e), span.row, e, f, value);
#pragma unroll
        for (int k = 0; k < ARITY; ++k) args[k] = a.prefix[(e * ARITY + k) * WIDTH + f];
#pragma unroll
        for (int j = 0; j < N_MESSAGES; ++j) args[ARITY + j] = value[kMessageSlot[j]];
        step_eval(args, rv);
        step_seed(radj, carried);
        step_back(rv, radj);
        step_args(radj, arg_adjoint);
#pragma unroll
        for (int k = 0; k < ARITY; ++k) carried[k] = arg_adjoint[k];
#pragma unroll
        for (int j = 0; j < N_MESSAGES; ++j)
          a.message_grads[((i64)j * a.num_edges + e) * WIDTH + f] = arg_adjoint[ARITY + j];
      }
    }
    if (LONG) __syncthreads();
  }
}

extern "C" __global__ void __launch_bounds__(THREADS) alg_fwd(const __grid_constant__ Args a) { algebra_forward<false>(a); }
extern "C" __global__ void __launch_bounds__(LONG_THREADS) alg_fwd_long(const __grid_constant__ Args a) { algebra_forward<true>(a); }
extern "C" __global__ void __launch_bounds__(THREADS) alg_bwd_messages(const __grid_constant__ Args a) { algebra_messages<false>(a); }
extern "C" __global__ void __launch_bounds__(LONG_THREADS) alg_bwd_messages_long(const __grid_constant__ Args a) { algebra_messages<true>(a); }
"""

_BINARY = {ep.OP_ADD: "__fadd_rn({a}, {b})", ep.OP_SUB: "__fsub_rn({a}, {b})", ep.OP_MUL: "__fmul_rn({a}, {b})",
           ep.OP_DIV: "__fdiv_rn({a}, {b})", ep.OP_MAX: "maximum_nan({a}, {b})"}


def _lanes(width: int) -> int:
    lanes = 1
    while lanes < 32 and lanes < width:
        lanes <<= 1
    return lanes


def _float_bits(value: float) -> str:
    """The exact float32 as a CUDA expression."""
    import struct

    return f"__int_as_float(0x{struct.unpack('<I', struct.pack('<f', float(value)))[0]:08x})"


def _forward_lines(ops, lhs, rhs, load, constant, target):
    """One statement per instruction: ``target[i] = ...``."""
    lines = []
    for i, (op, a, b) in enumerate(zip(ops, lhs, rhs)):
        if op == ep.OP_LOAD:
            lines.append(f"  {target}[{i}] = {load(a)};")
        elif op == ep.OP_CONST:
            lines.append(f"  {target}[{i}] = {constant(a)};")
        elif op in _BINARY:
            lines.append(f"  {target}[{i}] = " + _BINARY[op].format(a=f"{target}[{a}]", b=f"{target}[{b}]") + ";")
        elif op == ep.OP_EXP:
            lines.append(f"  {target}[{i}] = expf({target}[{a}]);")
        else:
            lines.append(f"  {target}[{i}] = -{target}[{a}];")
    return lines


def _reverse_lines(ops, lhs, rhs, value, adjoint):
    """The reverse sweep, last instruction first: pushes ``adjoint[i]`` down to the instruction's inputs."""
    lines = []
    for i in range(len(ops) - 1, -1, -1):
        op, a, b = ops[i], lhs[i], rhs[i]
        g = f"{adjoint}[{i}]"
        if op == ep.OP_ADD:
            lines.append(f"  {adjoint}[{a}] += {g}; {adjoint}[{b}] += {g};")
        elif op == ep.OP_SUB:
            lines.append(f"  {adjoint}[{a}] += {g}; {adjoint}[{b}] -= {g};")
        elif op == ep.OP_MUL:
            lines.append(f"  {{ const float gi = {g}; {adjoint}[{a}] += gi * {value}[{b}]; "
                         f"{adjoint}[{b}] += gi * {value}[{a}]; }}")
        elif op == ep.OP_DIV:
            lines.append(f"  {{ const float q = {g} / {value}[{b}]; {adjoint}[{a}] += q; "
                         f"{adjoint}[{b}] -= q * {value}[{i}]; }}")
        elif op == ep.OP_MAX:
            lines.append(f"  {{ const float gi = {g}, x = {value}[{a}], y = {value}[{b}]; "
                         f"{adjoint}[{a}] += x > y ? gi : (x == y ? 0.5f * gi : 0.0f); "
                         f"{adjoint}[{b}] += y > x ? gi : (x == y ? 0.5f * gi : 0.0f); }}")
        elif op == ep.OP_EXP:
            lines.append(f"  {adjoint}[{a}] += {g} * {value}[{i}];")
        elif op == ep.OP_NEG:
            lines.append(f"  {adjoint}[{a}] -= {g};")
    return lines


def _region_functions(name: str, region, n_args: int) -> str:
    """eval / out / seed / back / args of one reducer region (tiga.algebra.Region)."""
    n = len(region.ops)
    forward = _forward_lines(region.ops, region.lhs, region.rhs, lambda a: f"args[{a}]",
                             lambda c: _float_bits(region.constants[c]), "rv")
    reverse = _reverse_lines(region.ops, region.lhs, region.rhs, "rv", "radj")
    outs = [f"  out[{k}] = rv[{slot}];" for k, slot in enumerate(region.outs)]
    seed = ["#pragma unroll", f"  for (int i = 0; i < {n}; ++i) radj[i] = 0.0f;"] + \
           [f"  radj[{slot}] += out_adjoint[{k}];" for k, slot in enumerate(region.outs)]
    gather = []
    for argument in range(n_args):
        loads = [i for i, (op, a) in enumerate(zip(region.ops, region.lhs)) if op == ep.OP_LOAD and a == argument]
        gather.append(f"  arg_adjoint[{argument}] = " + (" + ".join(f"radj[{i}]" for i in loads) if loads else "0.0f") + ";")
    return "\n".join([
        f"__device__ __forceinline__ void {name}_eval(const float *args, float *rv) {{", *forward, "}",
        f"__device__ __forceinline__ void {name}_out(const float *rv, float *out) {{", *outs, "}",
        f"__device__ __forceinline__ void {name}_seed(float *radj, const float *out_adjoint) {{", *seed, "}",
        f"__device__ __forceinline__ void {name}_back(const float *rv, float *radj) {{", *reverse, "}",
        f"__device__ __forceinline__ void {name}_args(const float *radj, float *arg_adjoint) {{", *gather, "}"])


def generate_source(program: ep.EdgeProgram, width: int, moduli, reducer: int, rules=None, message_slots=None) -> str:
    """The CUDA source of the kernels specialised for this program: the six passes of a built-in
    reducer, or -- with ``rules`` (a ``tiga.algebra.Algebra``) and the message slots -- the algebra fold,
    its reverse sweep and the reverse passes seeded per edge."""
    n = len(program.ops)
    roles = [ep.ROLE_PARAM if o.role == "param" else ep._ROLES[o.role] for o in program.operands]
    load_slot = {a: i for i, (op, a) in enumerate(zip(program.ops, program.lhs)) if op == ep.OP_LOAD}

    def load(a):
        role, modulus = roles[a], int(moduli[a])
        entity = {ep.ROLE_SRC: "src", ep.ROLE_DST: "dst", ep.ROLE_EDGE: "edge", ep.ROLE_PARAM: "0"}[role]
        count = width if modulus == 0 else modulus
        offset = "f" if modulus == 0 else ("0" if modulus == 1 else f"f % {modulus}")
        return f"__ldg(a.in[{a}] + {entity} * {count} + {offset})"

    evaluate = _forward_lines(program.ops, program.lhs, program.rhs, load, lambda c: f"a.constants[{c}]", "value")
    sweep = _reverse_lines(program.ops, program.lhs, program.rhs, "value", "adjoint")
    count = len(program.operands)
    slots = tuple(message_slots) if message_slots is not None else (n - 1,)
    table = lambda values: ", ".join(str(int(v)) for v in values)      # noqa: E731
    defines = [
        f"#define WIDTH {int(width)}", f"#define LANES {_lanes(int(width))}", f"#define N_INSTR {n}",
        f"#define N_OPERANDS {count}", f"#define REDUCER {4 if rules is not None else int(reducer)}",
        f"#define N_MESSAGES {len(slots)}",
        # one CTA per long row: the more lane groups, the shorter the slice each walks (the library
        # launches the *_long kernels with the block size they declare)
        f"#define LONG_THREADS {512 if rules is not None else 1024}",
        f"__device__ constexpr int kRole[N_OPERANDS] = {{{table(roles)}}};",
        f"__device__ constexpr int kModulus[N_OPERANDS] = {{{table(moduli)}}};",
        f"__device__ constexpr int kLoadSlot[N_OPERANDS] = {{{table(load_slot[k] for k in range(count))}}};",
        f"__device__ constexpr int kMessageSlot[N_MESSAGES] = {{{table(slots)}}};",
        "#define constexpr_role_modulus(k) const int role = kRole[k], modulus = kModulus[k], load_slot = kLoadSlot[k]; "
        "(void)role; (void)modulus; (void)load_slot",
    ]
    functions = [
        "__device__ __forceinline__ void evaluate(const Args &a, i64 src, i64 dst, i64 edge, int f, float *value) {",
        *evaluate, "}",
        "__device__ __forceinline__ void sweep_back(const float *value, float *adjoint) {", *sweep, "}"]
    parts = ["\n".join(defines), _PRELUDE, "\n".join(functions), _KERNELS]
    if rules is not None:
        arity = rules.arity
        cases = " ".join(f"case {k}: return {_float_bits(v)};" for k, v in enumerate(rules.identity))
        algebra = [
            f"#define ARITY {arity}", f"#define N_STEP {len(rules.step.ops)}",
            f"#define N_COMBINE {len(rules.combine.ops)}", f"#define N_FINAL {len(rules.finalize.ops)}",
            f"__device__ __forceinline__ float identity_of(int k) {{ switch (k) {{ {cases} }} return 0.0f; }}",
            _region_functions("step", rules.step, arity + rules.num_messages),
            _region_functions("combine", rules.combine, 2 * arity),
            _region_functions("finalize", rules.finalize, arity)]
        parts += ["\n".join(algebra), _ALGEBRA_KERNELS]
    return "\n".join(parts)


class CompilerUnavailable(RuntimeError):
    """The NVRTC library could not be opened."""


class Module:
    """A compiled source (``tgb_jit_module``)."""

    def __init__(self, source: str):
        handle = ctypes.c_void_p()
        log = ctypes.create_string_buffer(16384)
        status = _native.lib().tgb_jit_build(source.encode(), ctypes.byref(handle), log, len(log))
        if status == 2:             # TGB_STATUS_UNSUPPORTED
            raise CompilerUnavailable("the NVRTC library (libnvrtc.so.12) could not be opened")
        if status != 0:
            raise RuntimeError("the generated edge-program source did not compile:\n" + log.value.decode(errors="replace"))
        self.handle = handle
        self.source = source

    def __del__(self):
        if sys is None or sys.is_finalizing():      # process exit releases the module with the context
            return
        try:
            if self.handle:
                _native.lib().tgb_jit_destroy(self.handle)
        except Exception:
            pass


_modules: dict = {}
_lock = threading.Lock()


def enabled() -> bool:
    """Generated kernels are the default; ``TGB_EDGE_JIT=0`` keeps every program on the interpreter."""
    return os.environ.get("TGB_EDGE_JIT", "1") != "0"


def module_for(program: ep.EdgeProgram, width: int, moduli, reducer: int, rules=None,
               message_slots=None) -> Module | None:
    """The module of this specialisation, compiled on first use; None when the runtime compiler is
    not available (the interpreting kernels then run the program)."""
    key = (program.key(), int(width), tuple(int(m) for m in moduli), int(reducer),
           None if rules is None else (rules.key(), tuple(message_slots)))
    with _lock:
        if key in _modules:
            return _modules[key]
    try:
        module = Module(generate_source(program, width, moduli, reducer, rules, message_slots))
    except CompilerUnavailable:
        module = None
    with _lock:
        _modules[key] = module
        if len(_modules) > 256:
            _modules.pop(next(iter(_modules)))
    return module


__all__ = ["CompilerUnavailable", "Module", "enabled", "generate_source", "module_for"]
