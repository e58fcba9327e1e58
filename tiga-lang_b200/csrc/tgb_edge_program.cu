// Generic edge programs: an element-wise edge expression, given as a small register program,
// evaluated per edge and feature element and folded over CSR rows; plus its reverse mode.
//
// Replaces the reference's generic CSR kernels (gf_csr_additive_tile with one row per program,
// lib/Target/Triton/Translate.cpp:2630-2783 with the expression emitter at :381-460, and
// gf_csr_scalar_reduce, :3452-3634, of walkerchi/TIGA-lang) and the Torch autograd replay behind them.
//
// One thread group of LANES lanes owns a row; lane l evaluates the feature elements l, l + LANES, ...
// one chunk after the other, walking the row's edges sequentially for each chunk, so a row is
// folded in edge order (the reference's left fold) and nothing is reduced with atomics.
//   forward           rows = destinations
//   backward (rows)   rows = destinations: cotangents of dst / edge / parameter operands
//   backward (sources) rows = sources over the plan's transposed relation: cotangents of src operands
// The interpreter costs ~10 instructions per program instruction; programs the library has a
// dedicated kernel for (weighted sums, attention) never come here.
#include <cstring>

#include "tgb_common.cuh"

namespace tgb {
namespace {

constexpr int kThreads = 128;
constexpr int kMaxI = TGB_EP_MAX_INSTRUCTIONS;
constexpr int kMaxO = TGB_EP_MAX_OPERANDS;

struct Operands {
  const float *ptr[kMaxO];
};
struct Sinks {
  float *ptr[kMaxO];
};

// One traversal: rows with their entries; entry -> (neighbour, edge id).
struct Walk {
  const void *ptr;        // row pointers
  const void *idx;        // neighbour per entry
  const uint32_t *eid;    // original edge id per entry, or null: entry index = edge id
  int ptr_bits, idx_bits;
  int64_t n_rows;
  const int32_t *order;   // plan row order: the n_long rows above the split threshold first
  int64_t n_long;
  int64_t split_threshold;
};

__device__ __forceinline__ int64_t load_index(const void *base, int bits, int64_t i) {
  return bits == 64 ? __ldg(static_cast<const int64_t *>(base) + i)
                    : (int64_t)__ldg(static_cast<const int32_t *>(base) + i);
}

// one arithmetic instruction (everything but LOAD and CONST)
__device__ __forceinline__ float apply_op(int op, float x, float y) {
  switch (op) {
    case TGB_EP_ADD: return __fadd_rn(x, y);
    case TGB_EP_SUB: return __fsub_rn(x, y);
    case TGB_EP_MUL: return __fmul_rn(x, y);
    case TGB_EP_DIV: return __fdiv_rn(x, y);
    case TGB_EP_MAX: return (x != x || y != y) ? __int_as_float(0x7fc00000) : fmaxf(x, y);   // torch.maximum: NaN wins
    case TGB_EP_EXP: return expf(x);
    default: return -x;   // TGB_EP_NEG
  }
}

// value[] of every instruction for one (source, destination, edge, element)
__device__ __forceinline__ void evaluate(const tgb_edge_program &p, const Operands &in, int64_t src, int64_t dst,
                                         int64_t edge, int f, float *value) {
  const int n = p.num_instructions;
  for (int i = 0; i < n; ++i) {
    const int a = p.a[i], b = p.b[i];
    float v;
    if (p.op[i] == TGB_EP_LOAD) {
      const int role = p.operand_role[a], m = p.operand_modulus[a];
      const int64_t entity = role == TGB_EP_ROLE_SRC ? src : role == TGB_EP_ROLE_DST ? dst
                             : role == TGB_EP_ROLE_EDGE ? edge : 0;
      const int count = m == 0 ? p.width : m;
      const int offset = m == 0 ? f : (m == 1 ? 0 : f % m);
      v = __ldg(in.ptr[a] + entity * count + offset);
    } else if (p.op[i] == TGB_EP_CONST) {
      v = p.constants[a];
    } else {
      v = apply_op(p.op[i], value[a], value[b]);
    }
    value[i] = v;
  }
}

// Pushes the adjoints of a program's instructions (tgb_edge_program or tgb_region) down to its
// leaves; the caller has put the seeds into adjoint[].
template <typename Program>
__device__ __forceinline__ void sweep_back(const Program &p, const float *value, float *adjoint) {
  for (int i = p.num_instructions - 1; i >= 0; --i) {
    const float gi = adjoint[i];
    const int a = p.a[i], b = p.b[i];
    switch (p.op[i]) {
      case TGB_EP_ADD: adjoint[a] += gi; adjoint[b] += gi; break;
      case TGB_EP_SUB: adjoint[a] += gi; adjoint[b] -= gi; break;
      case TGB_EP_MUL: adjoint[a] += gi * value[b]; adjoint[b] += gi * value[a]; break;
      case TGB_EP_DIV: {
        const float q = gi / value[b];
        adjoint[a] += q;
        adjoint[b] -= q * value[i];
        break;
      }
      case TGB_EP_MAX: {     // the larger operand takes the cotangent, equal operands share it
        const float x = value[a], y = value[b];
        adjoint[a] += x > y ? gi : (x == y ? 0.5f * gi : 0.0f);
        adjoint[b] += y > x ? gi : (x == y ? 0.5f * gi : 0.0f);
        break;
      }
      case TGB_EP_EXP: adjoint[a] += gi * value[i]; break;
      case TGB_EP_NEG: adjoint[a] -= gi; break;
      default: break;        // LOAD: a sink; CONST: nothing
    }
  }
}

// adjoint[] of every instruction given the cotangent g of the message (the last instruction)
__device__ __forceinline__ void reverse_sweep(const tgb_edge_program &p, const float *value, float g, float *adjoint) {
  const int n = p.num_instructions;
  for (int i = 0; i < n; ++i) adjoint[i] = 0.0f;
  adjoint[n - 1] = g;
  sweep_back(p, value, adjoint);
}

// Message cotangents given per edge and message slot (the reverse mode of a user algebra hands them
// over this way): [count][edges][width].
struct Seeds {
  const float *base;
  int64_t edges;
  int count;
  uint8_t slot[TGB_ALG_MAX_MESSAGES];
};
constexpr int kReducerSeeded = -1;     // k_edge_program_bwd: take the message cotangents from Seeds

template <int LANES>
__device__ __forceinline__ unsigned group_mask() {
  return LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u) << ((threadIdx.x & 31) / LANES * LANES);
}

template <int LANES>
__device__ __forceinline__ float group_sum(float v, unsigned mask) {
#pragma unroll
  for (int offset = LANES / 2; offset > 0; offset >>= 1) v += __shfl_xor_sync(mask, v, offset, LANES);
  return v;
}

// LONG = false: one lane group per row, rows longer than the plan's split threshold are left to the
// LONG launch.  LONG = true: one CTA per long row (blockIdx.x-th entry of the plan's row order, which
// lists the long rows first); its lane groups fold contiguous slices of the row's edges and the slices'
// partial results are combined in slice order through shared memory (deterministic).
constexpr int kLongThreads = 256;

// What the forward keeps per (row, element) for the reverse mode of the reducers whose message
// cotangent depends on the other messages of the row:
//   MAX   index = entry (CSR position) of the first message that reached the row's maximum, -1 if none did
//   PROD  value = product of the row's messages with every zero replaced by one, index = number of zeros
struct Saved {
  float *value;
  int32_t *index;
};

__device__ __forceinline__ float max_step(float state, float m) {      // NaN poisons the state
  return (state != state || m != m) ? __int_as_float(0x7fc00000) : fmaxf(state, m);
}
__device__ __forceinline__ bool max_takes(float state, float m) {      // does m replace the state's winner?
  return state == state && (m != m || m > state);
}

template <int LANES, bool LONG>
__global__ void __launch_bounds__(LONG ? kLongThreads : kThreads)
k_edge_program_fwd(const __grid_constant__ tgb_edge_program p, Operands in, Walk w, int reducer, float identity,
                   float *__restrict__ out, Saved saved) {
  constexpr int kGroups = (LONG ? kLongThreads : kThreads) / LANES;
  __shared__ float part[LONG ? kLongThreads : 1];
  __shared__ float part_masked[LONG ? kLongThreads : 1];
  __shared__ int32_t part_mark[LONG ? kLongThreads : 1];
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  int64_t row;
  if (LONG) {
    row = __ldg(w.order + blockIdx.x);
  } else {               // the rows below the split threshold, in the plan's bucket order
    const int64_t position = w.n_long + (int64_t)blockIdx.x * kGroups + group;
    if (position >= w.n_rows) return;
    row = __ldg(w.order + position);
  }
  int64_t begin = load_index(w.ptr, w.ptr_bits, row), end = load_index(w.ptr, w.ptr_bits, row + 1);
  const int64_t degree = end - begin;
  if (LONG) {
    const int64_t slice = (degree + kGroups - 1) / kGroups;
    begin = begin + group * slice;
    end = begin + slice < end ? begin + slice : end;
  }
  const bool is_max = reducer == TGB_REDUCER_MAX, is_prod = reducer == TGB_REDUCER_PROD;
  float value[kMaxI];
  for (int f0 = 0; f0 < p.width; f0 += LANES) {
    const int f = f0 + lane;
    // the fold starts from the identity; the slices of a long row start from the neutral element
    float acc = is_max ? identity : is_prod ? (LONG ? 1.0f : identity)
                                            : ((LONG || reducer == TGB_REDUCER_MEAN) ? 0.0f : identity);
    float masked = acc;                 // PROD only
    int32_t mark = is_max ? -1 : 0;     // MAX: winning entry; PROD: zeros seen
    if (f < p.width) {
      for (int64_t e = begin; e < end; ++e) {
        evaluate(p, in, load_index(w.idx, w.idx_bits, e), row, e, f, value);
        const float m = value[p.num_instructions - 1];
        if (is_max) {
          if (max_takes(acc, m)) mark = (int32_t)e;
          acc = max_step(acc, m);
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
      if (group == 0 && f < p.width) {
        // SUM / PROD: identity, then the slices in order; MAX / MEAN: the first slice, then the others
        const bool from_identity = reducer == TGB_REDUCER_SUM || is_prod;
        float total = from_identity ? identity : acc;
        float masked_total = identity;
        int32_t mark_total = is_prod ? 0 : mark;
        for (int g = from_identity ? 0 : 1; g < kGroups; ++g) {
          const float q = part[g * LANES + lane];
          if (is_max) {
            if (max_takes(total, q)) mark_total = part_mark[g * LANES + lane];
            total = max_step(total, q);
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
    if (f < p.width) {
      if (reducer == TGB_REDUCER_MEAN) acc = __fdiv_rn(acc, (float)degree);
      out[row * p.width + f] = acc;
      if (saved.value) saved.value[row * p.width + f] = masked;
      if (saved.index) saved.index[row * p.width + f] = mark;
    }
  }
}

// Reverse mode over one traversal.  The pass owns, per ROW, the operands of its own side (dst and
// tensor parameters in the destination-major pass, src in the source-major pass); EDGE operands are
// written per entry by the destination-major pass.
template <int LANES, bool SOURCE_MAJOR, bool LONG>
__global__ void __launch_bounds__(LONG ? kLongThreads : kThreads)
k_edge_program_bwd(const __grid_constant__ tgb_edge_program p, Operands in, Sinks sinks, Walk w, int reducer,
                   const void *__restrict__ degree_ptr, int degree_bits, const float *__restrict__ dy,
                   const float *__restrict__ saved_value, const int32_t *__restrict__ saved_index, Seeds seeds) {
  constexpr int kGroups = (LONG ? kLongThreads : kThreads) / LANES;
  __shared__ float part_full[LONG ? kMaxO * kLongThreads : 1];     // [operand][group][lane]
  __shared__ float part_scalar[LONG ? kMaxO * kLongThreads : 1];   // [operand][group]
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  int64_t row;
  if (LONG) {
    row = __ldg(w.order + blockIdx.x);
  } else {
    const int64_t position = w.n_long + (int64_t)blockIdx.x * kGroups + group;
    if (position >= w.n_rows) return;
    row = __ldg(w.order + position);
  }
  const unsigned mask = group_mask<LANES>();
  int64_t begin = load_index(w.ptr, w.ptr_bits, row), end = load_index(w.ptr, w.ptr_bits, row + 1);
  if (LONG) {            // contiguous slices of the row's entries, one per lane group
    const int64_t slice = (end - begin + kGroups - 1) / kGroups;
    begin = begin + group * slice;
    end = begin + slice < end ? begin + slice : end;
  }
  // does this pass own operand k per row?
  auto row_owned = [&](int k) {
    if (k >= p.num_operands || sinks.ptr[k] == nullptr) return false;
    const int role = p.operand_role[k];
    return role != TGB_EP_ROLE_EDGE && (role == TGB_EP_ROLE_SRC) == SOURCE_MAJOR;
  };
  float value[kMaxI], adjoint[kMaxI];
  float scalar_total[kMaxO];          // per-lane partial sums of the row-owned operands with one element per entity
#pragma unroll
  for (int k = 0; k < kMaxO; ++k) scalar_total[k] = 0.0f;
  // the group runs ceil(width / LANES) chunks together, so that its shuffles see all lanes
  const int chunks = (p.width + LANES - 1) / LANES;
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int f = chunk * LANES + lane;
    const bool live = f < p.width;
    float full_total[kMaxO];
#pragma unroll
    for (int k = 0; k < kMaxO; ++k) full_total[k] = 0.0f;
    for (int64_t t = begin; t < end; ++t) {
      const int64_t other = load_index(w.idx, w.idx_bits, t);
      const int64_t edge = w.eid ? (int64_t)__ldg(w.eid + t) : t;
      const int64_t src = SOURCE_MAJOR ? row : other, dst = SOURCE_MAJOR ? other : row;
      if (live) {
        evaluate(p, in, src, dst, edge, f, value);
        // the message's cotangent: what the reducer passes down from the row's cotangent
        float g = reducer == kReducerSeeded ? 0.0f : __ldg(dy + dst * p.width + f);
        if (reducer == TGB_REDUCER_MEAN) {
          const int64_t degree = load_index(degree_ptr, degree_bits, dst + 1) - load_index(degree_ptr, degree_bits, dst);
          g = g / (float)degree;
        } else if (reducer == TGB_REDUCER_MAX) {      // the first message that reached the maximum takes it all
          if (__ldg(saved_index + dst * p.width + f) != (int32_t)edge) g = 0.0f;
        } else if (reducer == TGB_REDUCER_PROD) {     // g times the product of the row's other messages, zero-safe
          const float m = value[p.num_instructions - 1];
          const float others = __ldg(saved_value + dst * p.width + f);
          const int32_t zeros = __ldg(saved_index + dst * p.width + f);
          g = zeros == 0 ? __fdiv_rn(__fmul_rn(g, others), m)
                         : (zeros == 1 && m == 0.0f) ? __fmul_rn(g, others) : 0.0f;
        }
        if (reducer == kReducerSeeded) {
          for (int i = 0; i < p.num_instructions; ++i) adjoint[i] = 0.0f;
          for (int j = 0; j < seeds.count; ++j)
            adjoint[seeds.slot[j]] += __ldg(seeds.base + ((int64_t)j * seeds.edges + edge) * p.width + f);
          sweep_back(p, value, adjoint);
        } else {
          reverse_sweep(p, value, g, adjoint);
        }
      }
      // every operand is loaded by exactly one instruction: its adjoint is the operand's cotangent
      for (int i = 0; i < p.num_instructions; ++i) {
        if (p.op[i] != TGB_EP_LOAD) continue;
        const int k = p.a[i];
        float *sink = sinks.ptr[k];
        if (sink == nullptr) continue;
        const int role = p.operand_role[k];
        const bool full = p.operand_modulus[k] == 0 || p.width == 1;
        const float gk = live ? adjoint[i] : 0.0f;
        if (role == TGB_EP_ROLE_EDGE) {
          if (SOURCE_MAJOR) continue;
          if (full) {
            if (live) sink[edge * p.width + f] = gk;
          } else {             // one value per edge: lanes and chunks add up, chunk after chunk by lane 0
            const float total = group_sum<LANES>(gk, mask);
            if (lane == 0) sink[edge] = chunk == 0 ? total : sink[edge] + total;
          }
        } else if ((role == TGB_EP_ROLE_SRC) == SOURCE_MAJOR) {
#pragma unroll
          for (int q = 0; q < kMaxO; ++q)
            if (q == k) {
              if (full) full_total[q] += gk; else scalar_total[q] += gk;
            }
        }
      }
    }
    if (LONG) {          // the slices' sums of this chunk, added in slice order by the first group
#pragma unroll
      for (int k = 0; k < kMaxO; ++k) part_full[k * kLongThreads + threadIdx.x] = full_total[k];
      __syncthreads();
      if (group == 0) {
#pragma unroll
        for (int k = 0; k < kMaxO; ++k) {
          float total = 0.0f;
          for (int g = 0; g < kGroups; ++g) total += part_full[k * kLongThreads + g * LANES + lane];
          full_total[k] = total;
        }
      }
      __syncthreads();
    }
    if (!LONG || group == 0) {
#pragma unroll
      for (int k = 0; k < kMaxO; ++k) {
        if (!row_owned(k)) continue;
        const bool full = p.operand_modulus[k] == 0 || p.width == 1;
        if (full && live) sinks.ptr[k][row * p.width + f] = full_total[k];
      }
    }
  }
  if constexpr (LONG) {
#pragma unroll
    for (int k = 0; k < kMaxO; ++k) {
      const float total = group_sum<LANES>(scalar_total[k], mask);
      if (lane == 0) part_scalar[k * kLongThreads + group] = total;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
      for (int k = 0; k < kMaxO; ++k) {
        if (!row_owned(k) || p.operand_modulus[k] == 0 || p.width == 1) continue;
        float total = 0.0f;
        for (int g = 0; g < kGroups; ++g) total += part_scalar[k * kLongThreads + g];
        sinks.ptr[k][row] = total;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < kMaxO; ++k) {
      if (!row_owned(k)) continue;
      const bool full = p.operand_modulus[k] == 0 || p.width == 1;
      if (full) continue;
      const float total = group_sum<LANES>(scalar_total[k], mask);
      if (lane == 0) sinks.ptr[k][row] = total;
    }
  }
}

// out[c] = sum_r partial[r, c]: 32 columns x 8 row strips per block, strips added in order
__global__ void __launch_bounds__(256)
k_column_sum(const float *__restrict__ partial, int64_t rows, int64_t cols, float *__restrict__ out) {
  __shared__ float strip[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + tx;
  float acc = 0.0f;
  if (c < cols)
    for (int64_t r = ty; r < rows; r += 8) acc += __ldg(partial + r * cols + c);
  strip[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float total = strip[0][tx];
#pragma unroll
    for (int s = 1; s < 8; ++s) total += strip[s][tx];
    out[c] = total;
  }
}

int lanes_for_width(int width) {
  int lanes = 1;
  while (lanes < 32 && lanes < width) lanes <<= 1;
  return lanes;
}

int32_t check_program(const tgb_csr_plan *plan, const tgb_edge_program *p, const void *const *operands) {
  if (!plan || !p || !operands) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null argument");
  if (plan->fwd.eid) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "edge programs do not take a plan with an edge map");
  if (p->num_instructions < 1 || p->num_instructions > kMaxI || p->num_operands < 1 || p->num_operands > kMaxO)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "program size out of range");
  if (p->width < 1) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "message width must be positive");
  int loads[kMaxO] = {0};
  for (int i = 0; i < p->num_instructions; ++i) {
    const int op = p->op[i];
    if (op > TGB_EP_NEG) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown opcode %d", op);
    if (op == TGB_EP_LOAD) {
      if (p->a[i] >= p->num_operands) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "operand index out of range");
      if (++loads[p->a[i]] > 1) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "an operand must be loaded by one instruction");
    } else if (op == TGB_EP_CONST) {
      if (p->a[i] >= TGB_EP_MAX_CONSTANTS) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "constant index out of range");
    } else {
      const bool binary = op >= TGB_EP_ADD && op <= TGB_EP_MAX;
      if (p->a[i] >= i || (binary && p->b[i] >= i))
        TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "instruction %d reads a later value", i);
    }
  }
  for (int k = 0; k < p->num_operands; ++k) {
    if (!operands[k]) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null operand %d", k);
    const int m = p->operand_modulus[k];
    if (m < 0 || (m > 1 && p->width % m != 0)) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "operand %d: bad modulus", k);
    if (p->operand_role[k] < 0 || p->operand_role[k] > TGB_EP_ROLE_PARAM)
      TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "operand %d: bad role", k);
  }
  return TGB_STATUS_OK;
}

Walk forward_walk(const tgb_csr_plan *plan) {
  return Walk{plan->fwd.ptr, plan->fwd.idx, nullptr, plan->fwd.ptr_bits, plan->fwd.idx_bits, plan->num_dst,
              plan->fwd.order, plan->fwd.n_long, kSplitThreshold};
}

}  // namespace
}  // namespace tgb

using namespace tgb;

#define TGB_EP_LANES(lanes, CALL)       \
  switch (lanes) {                      \
    case 1: CALL(1); break;             \
    case 2: CALL(2); break;             \
    case 4: CALL(4); break;             \
    case 8: CALL(8); break;             \
    case 16: CALL(16); break;           \
    default: CALL(32); break;           \
  }

extern "C" int32_t tgb_edge_program_fwd(const tgb_csr_plan *plan, const tgb_edge_program *program,
                                        const void *const *operands, int32_t reducer, float identity, void *out,
                                        void *saved_value, void *saved_index, uint64_t stream) {
  const int32_t status = check_program(plan, program, operands);
  if (status != TGB_STATUS_OK) return status;
  if (reducer < TGB_REDUCER_SUM || reducer > TGB_REDUCER_PROD) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown reducer");
  if (plan->num_dst == 0) return TGB_STATUS_OK;
  if (!out) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null output");
  if (saved_index && plan->num_edges >= ((int64_t)1 << 31))
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the saved entry index is 32 bits wide");
  const Saved saved{reducer == TGB_REDUCER_PROD ? static_cast<float *>(saved_value) : nullptr,
                    reducer == TGB_REDUCER_PROD || reducer == TGB_REDUCER_MAX ? static_cast<int32_t *>(saved_index)
                                                                                : nullptr};
  Operands in;
  for (int k = 0; k < kMaxO; ++k) in.ptr[k] = k < program->num_operands ? static_cast<const float *>(operands[k]) : nullptr;
  const Walk w = forward_walk(plan);
  const int lanes = lanes_for_width(program->width);
  const unsigned blocks = (unsigned)ceil_div(plan->num_dst * lanes, kThreads);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define TGB_FWD(L)                                                                                          \
  k_edge_program_fwd<L, false><<<blocks, kThreads, 0, st>>>(*program, in, w, reducer, identity,             \
                                                            static_cast<float *>(out), saved);              \
  if (w.n_long > 0)                                                                                         \
    k_edge_program_fwd<L, true><<<(unsigned)w.n_long, kLongThreads, 0, st>>>(*program, in, w, reducer, identity, \
                                                                             static_cast<float *>(out), saved)
  TGB_EP_LANES(lanes, TGB_FWD)
#undef TGB_FWD
  TGB_LAUNCHED();
  if (w.n_long > 0) TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

namespace {

int32_t backward(bool source_major, const tgb_csr_plan *plan, const tgb_edge_program *program,
                 const void *const *operands, int32_t reducer, const void *dy, void *const *grads,
                 const void *saved_value, const void *saved_index, uint64_t stream,
                 Seeds seeds = Seeds{nullptr, 0, 0, {0, 0, 0, 0}}) {
  const int32_t status = check_program(plan, program, operands);
  if (status != TGB_STATUS_OK) return status;
  if (reducer == kReducerSeeded ? seeds.base == nullptr : (reducer < TGB_REDUCER_SUM || reducer > TGB_REDUCER_PROD))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown reducer");
  if ((reducer == TGB_REDUCER_MAX || reducer == TGB_REDUCER_PROD) && !saved_index)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "this reducer's reverse mode needs what the forward saved (saved_index)");
  if (reducer == TGB_REDUCER_PROD && !saved_value)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "the product reducer's reverse mode needs saved_value");
  if (!dy || !grads) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null cotangent");
  if (source_major && !(plan->flags & TGB_PLAN_TRANSPOSE))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "the source-major pass needs a plan with the transposed relation");
  Operands in;
  Sinks sinks;
  bool any = false;
  for (int k = 0; k < kMaxO; ++k) {
    in.ptr[k] = k < program->num_operands ? static_cast<const float *>(operands[k]) : nullptr;
    sinks.ptr[k] = nullptr;
    if (k >= program->num_operands || !grads[k]) continue;
    const int role = program->operand_role[k];
    const bool mine = source_major ? role == TGB_EP_ROLE_SRC : role != TGB_EP_ROLE_SRC;
    if (!mine) continue;
    if (program->operand_modulus[k] > 1)
      TGB_FAIL(TGB_STATUS_UNSUPPORTED, "operand %d broadcasts along trailing dimensions: no cotangent kernel", k);
    sinks.ptr[k] = static_cast<float *>(grads[k]);
    any = true;
  }
  if (!any) return TGB_STATUS_OK;
  Walk w = forward_walk(plan);
  if (source_major) w = Walk{plan->bwd.ptr, plan->bwd.idx, plan->bwd.eid, plan->bwd.ptr_bits, plan->bwd.idx_bits,
                             plan->num_src, plan->bwd.order, plan->bwd.n_long, kSplitThreshold};
  if (w.n_rows == 0) return TGB_STATUS_OK;
  const int lanes = lanes_for_width(program->width);
  const unsigned blocks = (unsigned)ceil_div(w.n_rows * lanes, kThreads);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float *sv = static_cast<const float *>(saved_value);
  const int32_t *si = static_cast<const int32_t *>(saved_index);
#define TGB_BWD(L)                                                                                            \
  if (source_major) {                                                                                         \
    k_edge_program_bwd<L, true, false><<<blocks, kThreads, 0, st>>>(*program, in, sinks, w, reducer,          \
        plan->fwd.ptr, plan->fwd.ptr_bits, static_cast<const float *>(dy), sv, si, seeds);                         \
    if (w.n_long > 0)                                                                                         \
      k_edge_program_bwd<L, true, true><<<(unsigned)w.n_long, kLongThreads, 0, st>>>(*program, in, sinks, w,  \
          reducer, plan->fwd.ptr, plan->fwd.ptr_bits, static_cast<const float *>(dy), sv, si, seeds);              \
  } else {                                                                                                    \
    k_edge_program_bwd<L, false, false><<<blocks, kThreads, 0, st>>>(*program, in, sinks, w, reducer,         \
        plan->fwd.ptr, plan->fwd.ptr_bits, static_cast<const float *>(dy), sv, si, seeds);                         \
    if (w.n_long > 0)                                                                                         \
      k_edge_program_bwd<L, false, true><<<(unsigned)w.n_long, kLongThreads, 0, st>>>(*program, in, sinks, w, \
          reducer, plan->fwd.ptr, plan->fwd.ptr_bits, static_cast<const float *>(dy), sv, si, seeds);              \
  }
  TGB_EP_LANES(lanes, TGB_BWD)
#undef TGB_BWD
  TGB_LAUNCHED();
  if (w.n_long > 0) TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

}  // namespace

extern "C" int32_t tgb_edge_program_bwd_rows(const tgb_csr_plan *plan, const tgb_edge_program *program,
                                             const void *const *operands, int32_t reducer, const void *dy,
                                             void *const *grads, const void *saved_value, const void *saved_index,
                                             uint64_t stream) {
  return backward(false, plan, program, operands, reducer, dy, grads, saved_value, saved_index, stream);
}

extern "C" int32_t tgb_edge_program_bwd_sources(const tgb_csr_plan *plan, const tgb_edge_program *program,
                                                const void *const *operands, int32_t reducer, const void *dy,
                                                void *const *grads, const void *saved_value,
                                                const void *saved_index, uint64_t stream) {
  return backward(true, plan, program, operands, reducer, dy, grads, saved_value, saved_index, stream);
}

// ---- the same three passes through a module generated for the program (tiga/edge_jit.py) ---------
namespace {

// The row-per-group kernel, then the kernel that gives every row above the split threshold a CTA of
// its own (launched with the block size it declares).  Running the second on a forked stream beside
// the first was measured: no gain, the long-row kernel is not a tail of a few CTAs.
int32_t launch_pair(tgb_jit_module *module, const char *short_kernel, uint32_t short_grid, const char *long_kernel,
                    int64_t n_long, const tgb_jit_edge_args *a, uint64_t stream) {
  int32_t rc = tgb_jit_launch(module, short_kernel, short_grid, kThreads, a, stream);
  if (rc == TGB_STATUS_OK && n_long > 0) rc = tgb_jit_launch(module, long_kernel, (uint32_t)n_long, 0, a, stream);
  return rc;
}

void fill_walk(tgb_jit_edge_args *a, const Walk &w) {
  a->ptr = w.ptr;
  a->idx = w.idx;
  a->eid = w.eid;
  a->order = w.order;
  a->n_rows = w.n_rows;
  a->n_long = w.n_long;
  a->split_threshold = w.split_threshold;
  a->ptr_bits = w.ptr_bits;
  a->idx_bits = w.idx_bits;
}

void fill_program(tgb_jit_edge_args *a, const tgb_csr_plan *plan, const tgb_edge_program *program,
                  const void *const *operands) {
  memset(a, 0, sizeof(*a));
  for (int k = 0; k < program->num_operands; ++k) a->in[k] = static_cast<const float *>(operands[k]);
  for (int c = 0; c < TGB_EP_MAX_CONSTANTS; ++c) a->constants[c] = program->constants[c];
  a->degree_ptr = plan->fwd.ptr;
  a->degree_bits = plan->fwd.ptr_bits;
}

}  // namespace

extern "C" int32_t tgb_edge_program_jit_fwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                            const tgb_edge_program *program, const void *const *operands,
                                            int32_t reducer, float identity, void *out, void *saved_value,
                                            void *saved_index, uint64_t stream) {
  const int32_t status = check_program(plan, program, operands);
  if (status != TGB_STATUS_OK) return status;
  if (!module) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null module");
  if (reducer < TGB_REDUCER_SUM || reducer > TGB_REDUCER_PROD) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown reducer");
  if (plan->num_dst == 0) return TGB_STATUS_OK;
  if (!out) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null output");
  if (saved_index && plan->num_edges >= ((int64_t)1 << 31))
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the saved entry index is 32 bits wide");
  tgb_jit_edge_args a;
  fill_program(&a, plan, program, operands);
  const Walk w = forward_walk(plan);
  fill_walk(&a, w);
  a.identity = identity;
  a.out = static_cast<float *>(out);
  a.saved_value = reducer == TGB_REDUCER_PROD ? static_cast<float *>(saved_value) : nullptr;
  a.saved_index = reducer == TGB_REDUCER_PROD || reducer == TGB_REDUCER_MAX ? static_cast<int32_t *>(saved_index)
                                                                            : nullptr;
  const int lanes = lanes_for_width(program->width);
  return launch_pair(module, "fwd", (uint32_t)ceil_div(plan->num_dst * lanes, kThreads), "fwd_long", w.n_long, &a,
                     stream);
}

namespace {

// The reverse pass of a generated module over one traversal; `seeds` != null: message cotangents
// per edge (user algebras) instead of a reducer rule.
int32_t jit_reverse(const tgb_csr_plan *plan, tgb_jit_module *module, const tgb_edge_program *program,
                    const void *const *operands, const void *dy, const void *seeds, void *const *grads,
                    const void *saved_value, const void *saved_index, int32_t source_major, uint64_t stream);

}  // namespace

extern "C" int32_t tgb_edge_program_jit_bwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                            const tgb_edge_program *program, const void *const *operands,
                                            int32_t reducer, const void *dy, void *const *grads,
                                            const void *saved_value, const void *saved_index,
                                            int32_t source_major, uint64_t stream) {
  const int32_t status = check_program(plan, program, operands);
  if (status != TGB_STATUS_OK) return status;
  if (reducer < TGB_REDUCER_SUM || reducer > TGB_REDUCER_PROD) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown reducer");
  if ((reducer == TGB_REDUCER_MAX || reducer == TGB_REDUCER_PROD) && !saved_index)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "this reducer's reverse mode needs what the forward saved (saved_index)");
  if (reducer == TGB_REDUCER_PROD && !saved_value)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "the product reducer's reverse mode needs saved_value");
  if (!dy) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null cotangent");
  return jit_reverse(plan, module, program, operands, dy, nullptr, grads, saved_value, saved_index, source_major,
                     stream);
}

namespace {

int32_t jit_reverse(const tgb_csr_plan *plan, tgb_jit_module *module, const tgb_edge_program *program,
                    const void *const *operands, const void *dy, const void *seeds, void *const *grads,
                    const void *saved_value, const void *saved_index, int32_t source_major, uint64_t stream) {
  if (!module) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null module");
  if (!grads) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null cotangent table");
  if (source_major && !(plan->flags & TGB_PLAN_TRANSPOSE))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "the source-major pass needs a plan with the transposed relation");
  tgb_jit_edge_args a;
  fill_program(&a, plan, program, operands);
  a.seeds = static_cast<const float *>(seeds);
  a.num_edges = plan->num_edges;
  bool any = false;
  for (int k = 0; k < program->num_operands; ++k) {
    if (!grads[k]) continue;
    const int role = program->operand_role[k];
    const bool mine = source_major ? role == TGB_EP_ROLE_SRC : role != TGB_EP_ROLE_SRC;
    if (!mine) continue;
    if (program->operand_modulus[k] > 1)
      TGB_FAIL(TGB_STATUS_UNSUPPORTED, "operand %d broadcasts along trailing dimensions: no cotangent kernel", k);
    a.sink[k] = static_cast<float *>(grads[k]);
    any = true;
  }
  if (!any) return TGB_STATUS_OK;
  Walk w = forward_walk(plan);
  if (source_major) w = Walk{plan->bwd.ptr, plan->bwd.idx, plan->bwd.eid, plan->bwd.ptr_bits, plan->bwd.idx_bits,
                             plan->num_src, plan->bwd.order, plan->bwd.n_long, kSplitThreshold};
  if (w.n_rows == 0) return TGB_STATUS_OK;
  fill_walk(&a, w);
  a.dy = static_cast<const float *>(dy);
  a.saved_value = const_cast<float *>(static_cast<const float *>(saved_value));
  a.saved_index = const_cast<int32_t *>(static_cast<const int32_t *>(saved_index));
  const int lanes = lanes_for_width(program->width);
  const uint32_t blocks = (uint32_t)ceil_div(w.n_rows * lanes, kThreads);
  return launch_pair(module, source_major ? "bwd_sources" : "bwd_rows", blocks,
                     source_major ? "bwd_sources_long" : "bwd_rows_long", w.n_long, &a, stream);
}

}  // namespace

extern "C" int32_t tgb_edge_algebra_jit_fwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                            const tgb_edge_program *program, const void *const *operands, void *out,
                                            uint64_t stream) {
  const int32_t status = check_program(plan, program, operands);
  if (status != TGB_STATUS_OK) return status;
  if (!module) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null module");
  if (plan->num_dst == 0) return TGB_STATUS_OK;
  if (!out) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null output");
  tgb_jit_edge_args a;
  fill_program(&a, plan, program, operands);
  const Walk w = forward_walk(plan);
  fill_walk(&a, w);
  a.out = static_cast<float *>(out);
  a.num_edges = plan->num_edges;
  const int lanes = lanes_for_width(program->width);
  return launch_pair(module, "alg_fwd", (uint32_t)ceil_div(plan->num_dst * lanes, kThreads), "alg_fwd_long", w.n_long,
                     &a, stream);
}

extern "C" int32_t tgb_edge_algebra_jit_bwd_messages(const tgb_csr_plan *plan, tgb_jit_module *module,
                                                     const tgb_edge_program *program, const void *const *operands,
                                                     const void *dy, void *prefix, void *message_grads,
                                                     uint64_t stream) {
  const int32_t status = check_program(plan, program, operands);
  if (status != TGB_STATUS_OK) return status;
  if (!module) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null module");
  if (plan->num_dst == 0 || plan->num_edges == 0) return TGB_STATUS_OK;
  if (!dy || !prefix || !message_grads) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  tgb_jit_edge_args a;
  fill_program(&a, plan, program, operands);
  const Walk w = forward_walk(plan);
  fill_walk(&a, w);
  a.dy = static_cast<const float *>(dy);
  a.prefix = static_cast<float *>(prefix);
  a.message_grads = static_cast<float *>(message_grads);
  a.num_edges = plan->num_edges;
  const int lanes = lanes_for_width(program->width);
  return launch_pair(module, "alg_bwd_messages", (uint32_t)ceil_div(plan->num_dst * lanes, kThreads),
                     "alg_bwd_messages_long", w.n_long, &a, stream);
}

extern "C" int32_t tgb_edge_algebra_jit_bwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                            const tgb_edge_program *program, const void *const *operands,
                                            const void *message_grads, void *const *grads, int32_t source_major,
                                            uint64_t stream) {
  const int32_t status = check_program(plan, program, operands);
  if (status != TGB_STATUS_OK) return status;
  if (!message_grads) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null message cotangents");
  return jit_reverse(plan, module, program, operands, message_grads, message_grads, grads, nullptr, nullptr,
                     source_major, stream);
}

extern "C" int32_t tgb_column_sum(const void *partial, int64_t rows, int64_t cols, void *out, uint64_t stream) {
  if (rows < 0 || cols < 1) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "invalid shape");
  if (!out || (rows > 0 && !partial)) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  k_column_sum<<<(unsigned)ceil_div(cols, 32), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const float *>(partial), rows, cols, static_cast<float *>(out));
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

// ===================================================================================================
// User algebras: the fold of a row is state = step(state, messages of the edge) from the identity,
// out = finalize(state), with step / combine / finalize given as register programs over arguments
// (the reference's captured reducer regions, python/tiga/compiler/reducer_capture.py:53-130, run by its
// generic tile gf_csr_algebra_tile, lib/Target/Triton/Translate.cpp:3065-3092).  Same row ownership as
// the kernels above: a lane group per row and element chunk, edges in order; a long row is folded in
// contiguous slices by one CTA and the slices are joined in order with `combine` (associativity is
// what the reducer declares; commutativity is not needed).
namespace tgb {
namespace {

constexpr int kMaxA = TGB_ALG_MAX_STATE;
constexpr int kMaxM = TGB_ALG_MAX_MESSAGES;
constexpr int kMaxR = TGB_ALG_MAX_INSTRUCTIONS;
constexpr int kMaxArgs = kMaxA + (kMaxA > kMaxM ? kMaxA : kMaxM);

__device__ __forceinline__ void region_eval(const tgb_region &r, const float *args, float *value) {
  for (int i = 0; i < r.num_instructions; ++i) {
    const int op = r.op[i], a = r.a[i], b = r.b[i];
    value[i] = op == TGB_EP_LOAD ? args[a] : op == TGB_EP_CONST ? r.constants[a] : apply_op(op, value[a], value[b]);
  }
}

// cotangents of the region's arguments given the cotangents of its outputs
__device__ __forceinline__ void region_reverse(const tgb_region &r, const float *value, const float *out_adjoint,
                                               int n_out, float *adjoint, float *arg_adjoint, int n_args) {
  for (int i = 0; i < r.num_instructions; ++i) adjoint[i] = 0.0f;
  for (int k = 0; k < n_out; ++k) adjoint[r.out[k]] += out_adjoint[k];
  sweep_back(r, value, adjoint);
  for (int k = 0; k < n_args; ++k) arg_adjoint[k] = 0.0f;
  for (int i = 0; i < r.num_instructions; ++i)
    if (r.op[i] == TGB_EP_LOAD) arg_adjoint[r.a[i]] += adjoint[i];
}

// state <- step(state, messages of one edge), given the edge program's values
__device__ __forceinline__ void fold_edge(const tgb_edge_algebra &alg, const float *edge_value, float *state,
                                          float *args, float *rv) {
  for (int k = 0; k < alg.arity; ++k) args[k] = state[k];
  for (int j = 0; j < alg.num_messages; ++j) args[alg.arity + j] = edge_value[alg.message_slot[j]];
  region_eval(alg.step, args, rv);
  for (int k = 0; k < alg.arity; ++k) state[k] = rv[alg.step.out[k]];
}

struct RowSpan {
  int64_t row, begin, end, degree, slice;
};

// The (slice of the) row this lane group works on; ok = false: nothing to do.
template <int LANES, bool LONG>
__device__ __forceinline__ bool row_span(const Walk &w, RowSpan *span) {
  constexpr int kGroups = (LONG ? kLongThreads : kThreads) / LANES;
  const int group = threadIdx.x / LANES;
  if (LONG) {
    span->row = __ldg(w.order + blockIdx.x);
  } else {
    const int64_t position = w.n_long + (int64_t)blockIdx.x * kGroups + group;
    if (position >= w.n_rows) return false;
    span->row = __ldg(w.order + position);
  }
  span->begin = load_index(w.ptr, w.ptr_bits, span->row);
  span->end = load_index(w.ptr, w.ptr_bits, span->row + 1);
  span->degree = span->end - span->begin;
  span->slice = 0;
  if (LONG) {
    span->slice = (span->degree + kGroups - 1) / kGroups;
    span->begin = span->begin + group * span->slice;
    span->end = span->begin + span->slice < span->end ? span->begin + span->slice : span->end;
  }
  return true;
}

template <int LANES, bool LONG>
__global__ void __launch_bounds__(LONG ? kLongThreads : kThreads)
k_edge_algebra_fwd(const __grid_constant__ tgb_edge_program p, const __grid_constant__ tgb_edge_algebra alg,
                   Operands in, Walk w, float *__restrict__ out) {
  constexpr int kGroups = (LONG ? kLongThreads : kThreads) / LANES;
  __shared__ float part[LONG ? kMaxA * kLongThreads : 1];        // [component][group][lane]: slice totals
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  RowSpan span;
  if (!row_span<LANES, LONG>(w, &span)) return;
  float value[kMaxI], rv[kMaxR], args[kMaxArgs], state[kMaxA];
  for (int f0 = 0; f0 < p.width; f0 += LANES) {
    const int f = f0 + lane;
    const bool live = f < p.width;
    for (int k = 0; k < alg.arity; ++k) state[k] = alg.identity[k];
    if (live) {
      for (int64_t e = span.begin; e < span.end; ++e) {
        evaluate(p, in, load_index(w.idx, w.idx_bits, e), span.row, e, f, value);
        fold_edge(alg, value, state, args, rv);
      }
    }
    if (LONG) {
      for (int k = 0; k < alg.arity; ++k) part[k * kLongThreads + threadIdx.x] = state[k];
      __syncthreads();
      if (group == 0 && live) {
        for (int k = 0; k < alg.arity; ++k) state[k] = alg.identity[k];
        for (int g = 0; g < kGroups && (int64_t)g * span.slice < span.degree; ++g) {     // the non-empty slices, in order
          for (int k = 0; k < alg.arity; ++k) {
            args[k] = state[k];
            args[alg.arity + k] = part[k * kLongThreads + g * LANES + lane];
          }
          region_eval(alg.combine, args, rv);
          for (int k = 0; k < alg.arity; ++k) state[k] = rv[alg.combine.out[k]];
        }
      }
      __syncthreads();
      if (group != 0) continue;
    }
    if (live) {
      region_eval(alg.finalize, state, rv);
      out[span.row * p.width + f] = rv[alg.finalize.out[0]];
    }
  }
}

// Cotangent of every message of every edge.  Sweep 1 folds the row and keeps the state BEFORE each
// edge in `prefix`; the cotangent of the final state comes from finalize; sweep 2 walks the row
// backwards through step, handing each edge its message cotangents and passing the state's on.
// Long rows: slice totals T_g, running joins R_{g+1} = combine(R_g, T_g) by the first group, the
// reverse of that chain gives every slice the cotangent of its total, and the slices then run their
// own sweep 2 (prefix states inside a slice are counted from the identity, as T_g is).
template <int LANES, bool LONG>
__global__ void __launch_bounds__(LONG ? kLongThreads : kThreads)
k_edge_algebra_bwd_messages(const __grid_constant__ tgb_edge_program p, const __grid_constant__ tgb_edge_algebra alg,
                            Operands in, Walk w, const float *__restrict__ dy, float *__restrict__ prefix,
                            float *__restrict__ message_grads, int64_t num_edges) {
  constexpr int kGroups = (LONG ? kLongThreads : kThreads) / LANES;
  __shared__ float part[LONG ? kMaxA * kLongThreads : 1];        // slice totals, then their cotangents
  __shared__ float joined[LONG ? kMaxA * kLongThreads : 1];      // R_g: the join of the slices before g
  const int lane = threadIdx.x % LANES, group = threadIdx.x / LANES;
  RowSpan span;
  if (!row_span<LANES, LONG>(w, &span)) return;
  const int arity = alg.arity;
  float value[kMaxI], rv[kMaxR], radj[kMaxR], args[kMaxArgs], arg_adjoint[kMaxArgs], state[kMaxA], carried[kMaxA];
  for (int f0 = 0; f0 < p.width; f0 += LANES) {
    const int f = f0 + lane;
    const bool live = f < p.width;
    for (int k = 0; k < arity; ++k) state[k] = alg.identity[k];
    if (live) {
      for (int64_t e = span.begin; e < span.end; ++e) {
        for (int k = 0; k < arity; ++k) prefix[(e * arity + k) * p.width + f] = state[k];
        evaluate(p, in, load_index(w.idx, w.idx_bits, e), span.row, e, f, value);
        fold_edge(alg, value, state, args, rv);
      }
    }
    for (int k = 0; k < arity; ++k) carried[k] = 0.0f;
    if (!LONG) {
      if (live) {
        const float g = __ldg(dy + span.row * p.width + f);
        region_eval(alg.finalize, state, rv);
        region_reverse(alg.finalize, rv, &g, 1, radj, carried, arity);
      }
    } else {
      for (int k = 0; k < arity; ++k) part[k * kLongThreads + threadIdx.x] = state[k];
      __syncthreads();
      if (group == 0 && live) {
        int used = 0;
        for (int k = 0; k < arity; ++k) state[k] = alg.identity[k];
        for (int g = 0; g < kGroups && (int64_t)g * span.slice < span.degree; ++g, ++used) {
          for (int k = 0; k < arity; ++k) {
            joined[k * kLongThreads + g * LANES + lane] = state[k];
            args[k] = state[k];
            args[arity + k] = part[k * kLongThreads + g * LANES + lane];
          }
          region_eval(alg.combine, args, rv);
          for (int k = 0; k < arity; ++k) state[k] = rv[alg.combine.out[k]];
        }
        const float g_row = __ldg(dy + span.row * p.width + f);
        region_eval(alg.finalize, state, rv);
        region_reverse(alg.finalize, rv, &g_row, 1, radj, carried, arity);
        for (int g = used - 1; g >= 0; --g) {
          for (int k = 0; k < arity; ++k) {
            args[k] = joined[k * kLongThreads + g * LANES + lane];
            args[arity + k] = part[k * kLongThreads + g * LANES + lane];
          }
          region_eval(alg.combine, args, rv);
          region_reverse(alg.combine, rv, carried, arity, radj, arg_adjoint, 2 * arity);
          for (int k = 0; k < arity; ++k) {
            carried[k] = arg_adjoint[k];
            part[k * kLongThreads + g * LANES + lane] = arg_adjoint[arity + k];
          }
        }
      }
      __syncthreads();
      for (int k = 0; k < arity; ++k) carried[k] = part[k * kLongThreads + threadIdx.x];
    }
    if (live) {
      for (int64_t e = span.end - 1; e >= span.begin; --e) {
        evaluate(p, in, load_index(w.idx, w.idx_bits, e), span.row, e, f, value);
        for (int k = 0; k < arity; ++k) args[k] = prefix[(e * arity + k) * p.width + f];
        for (int j = 0; j < alg.num_messages; ++j) args[arity + j] = value[alg.message_slot[j]];
        region_eval(alg.step, args, rv);
        region_reverse(alg.step, rv, carried, arity, radj, arg_adjoint, arity + alg.num_messages);
        for (int k = 0; k < arity; ++k) carried[k] = arg_adjoint[k];
        for (int j = 0; j < alg.num_messages; ++j)
          message_grads[((int64_t)j * num_edges + e) * p.width + f] = arg_adjoint[arity + j];
      }
    }
    if (LONG) __syncthreads();       // `part` is written again by the next chunk
  }
}

int32_t check_region(const tgb_region &r, int n_args, int n_out, const char *name) {
  if (r.num_instructions < 1 || r.num_instructions > kMaxR)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "%s: region size out of range", name);
  for (int i = 0; i < r.num_instructions; ++i) {
    const int op = r.op[i];
    if (op > TGB_EP_NEG) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "%s: unknown opcode %d", name, op);
    if (op == TGB_EP_LOAD) {
      if (r.a[i] >= n_args) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "%s: argument index out of range", name);
    } else if (op == TGB_EP_CONST) {
      if (r.a[i] >= TGB_ALG_MAX_CONSTANTS) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "%s: constant index out of range", name);
    } else {
      const bool binary = op >= TGB_EP_ADD && op <= TGB_EP_MAX;
      if (r.a[i] >= i || (binary && r.b[i] >= i))
        TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "%s: instruction %d reads a later value", name, i);
    }
  }
  for (int k = 0; k < n_out; ++k)
    if (r.out[k] >= r.num_instructions) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "%s: output %d out of range", name, k);
  return TGB_STATUS_OK;
}

int32_t check_algebra(const tgb_edge_program *p, const tgb_edge_algebra *alg) {
  if (!alg) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null algebra");
  if (alg->arity < 1 || alg->arity > kMaxA || alg->num_messages < 1 || alg->num_messages > kMaxM)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "algebra: state or message count out of range");
  for (int j = 0; j < alg->num_messages; ++j)
    if (alg->message_slot[j] >= p->num_instructions) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "algebra: message slot out of range");
  int32_t status = check_region(alg->step, alg->arity + alg->num_messages, alg->arity, "step");
  if (status == TGB_STATUS_OK) status = check_region(alg->combine, 2 * alg->arity, alg->arity, "combine");
  if (status == TGB_STATUS_OK) status = check_region(alg->finalize, alg->arity, 1, "finalize");
  return status;
}

Operands operand_table(const tgb_edge_program *program, const void *const *operands) {
  Operands in;
  for (int k = 0; k < kMaxO; ++k) in.ptr[k] = k < program->num_operands ? static_cast<const float *>(operands[k]) : nullptr;
  return in;
}

Seeds message_seeds(const tgb_csr_plan *plan, const tgb_edge_algebra *alg, const void *message_grads) {
  Seeds seeds{static_cast<const float *>(message_grads), plan->num_edges, alg->num_messages, {0, 0, 0, 0}};
  for (int j = 0; j < alg->num_messages; ++j) seeds.slot[j] = alg->message_slot[j];
  return seeds;
}

}  // namespace
}  // namespace tgb

extern "C" int32_t tgb_edge_algebra_fwd(const tgb_csr_plan *plan, const tgb_edge_program *program,
                                        const tgb_edge_algebra *algebra, const void *const *operands, void *out,
                                        uint64_t stream) {
  int32_t status = check_program(plan, program, operands);
  if (status == TGB_STATUS_OK) status = check_algebra(program, algebra);
  if (status != TGB_STATUS_OK) return status;
  if (plan->num_dst == 0) return TGB_STATUS_OK;
  if (!out) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null output");
  const Operands in = operand_table(program, operands);
  const Walk w = forward_walk(plan);
  const int lanes = lanes_for_width(program->width);
  const unsigned blocks = (unsigned)ceil_div(plan->num_dst * lanes, kThreads);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define TGB_FWD(L)                                                                                                  \
  k_edge_algebra_fwd<L, false><<<blocks, kThreads, 0, st>>>(*program, *algebra, in, w, static_cast<float *>(out)); \
  if (w.n_long > 0)                                                                                                 \
    k_edge_algebra_fwd<L, true><<<(unsigned)w.n_long, kLongThreads, 0, st>>>(*program, *algebra, in, w,            \
                                                                             static_cast<float *>(out))
  TGB_EP_LANES(lanes, TGB_FWD)
#undef TGB_FWD
  TGB_LAUNCHED();
  if (w.n_long > 0) TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_edge_algebra_bwd_messages(const tgb_csr_plan *plan, const tgb_edge_program *program,
                                                 const tgb_edge_algebra *algebra, const void *const *operands,
                                                 const void *dy, void *prefix, void *message_grads,
                                                 uint64_t stream) {
  int32_t status = check_program(plan, program, operands);
  if (status == TGB_STATUS_OK) status = check_algebra(program, algebra);
  if (status != TGB_STATUS_OK) return status;
  if (plan->num_dst == 0 || plan->num_edges == 0) return TGB_STATUS_OK;
  if (!dy || !prefix || !message_grads) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  const Operands in = operand_table(program, operands);
  const Walk w = forward_walk(plan);
  const int lanes = lanes_for_width(program->width);
  const unsigned blocks = (unsigned)ceil_div(plan->num_dst * lanes, kThreads);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define TGB_BWD(L)                                                                                                   \
  k_edge_algebra_bwd_messages<L, false><<<blocks, kThreads, 0, st>>>(                                                \
      *program, *algebra, in, w, static_cast<const float *>(dy), static_cast<float *>(prefix),                      \
      static_cast<float *>(message_grads), plan->num_edges);                                                        \
  if (w.n_long > 0)                                                                                                  \
    k_edge_algebra_bwd_messages<L, true><<<(unsigned)w.n_long, kLongThreads, 0, st>>>(                              \
        *program, *algebra, in, w, static_cast<const float *>(dy), static_cast<float *>(prefix),                    \
        static_cast<float *>(message_grads), plan->num_edges)
  TGB_EP_LANES(lanes, TGB_BWD)
#undef TGB_BWD
  TGB_LAUNCHED();
  if (w.n_long > 0) TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_edge_algebra_bwd_rows(const tgb_csr_plan *plan, const tgb_edge_program *program,
                                             const tgb_edge_algebra *algebra, const void *const *operands,
                                             const void *message_grads, void *const *grads, uint64_t stream) {
  if (!plan || !program) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null argument");
  const int32_t status = check_algebra(program, algebra);
  if (status != TGB_STATUS_OK) return status;
  if (!message_grads) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null message cotangents");
  return backward(false, plan, program, operands, kReducerSeeded, message_grads, grads, nullptr, nullptr, stream,
                  message_seeds(plan, algebra, message_grads));
}

extern "C" int32_t tgb_edge_algebra_bwd_sources(const tgb_csr_plan *plan, const tgb_edge_program *program,
                                                const tgb_edge_algebra *algebra, const void *const *operands,
                                                const void *message_grads, void *const *grads, uint64_t stream) {
  if (!plan || !program) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null argument");
  const int32_t status = check_algebra(program, algebra);
  if (status != TGB_STATUS_OK) return status;
  if (!message_grads) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null message cotangents");
  return backward(true, plan, program, operands, kReducerSeeded, message_grads, grads, nullptr, nullptr, stream,
                  message_seeds(plan, algebra, message_grads));
}
