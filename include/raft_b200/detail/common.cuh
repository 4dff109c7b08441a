// Device-side building blocks shared by every reduction kernel of this library:
// 16-byte vector loads, word-wise warp shuffles for arbitrary accumulator types,
// the accumulator states (generic / compensated / widened), and the transposing
// sub-warp reduction that turns U per-lane partials into U finished rows with
// U-1 + log2(G/U) exchanges instead of U*log2(G).
//
// Everything here is header-only so that the same templates are instantiated
//  (1) inside the shared library for the operator combinations the C ABI names, and
//  (2) inside a caller's translation unit when the drop-in raft::linalg headers are
//      given a functor the C ABI cannot name (a device lambda, a user struct).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <type_traits>

namespace raft_b200 {
namespace detail {

#define B2R_DI __device__ __forceinline__
#define B2R_HDI __host__ __device__ __forceinline__

constexpr int kWarp = 32;

template <typename T>
B2R_HDI constexpr T ceil_div(T a, T b)
{
  return (a + b - 1) / b;
}

B2R_HDI constexpr int ilog2_floor(unsigned v)
{
  int r = 0;
  while (v > 1u) {
    v >>= 1;
    ++r;
  }
  return r;
}

B2R_HDI constexpr unsigned next_pow2(unsigned v)
{
  unsigned p = 1;
  while (p < v)
    p <<= 1;
  return p;
}

// ---------------------------------------------------------------------------------------
// 16-byte global loads. `VecOf<T, V>` is V consecutive elements of T moved by ONE load
// instruction when V*sizeof(T) is 4, 8 or 16 bytes.
// ---------------------------------------------------------------------------------------
template <typename T, int V>
struct alignas(sizeof(T) * V) VecOf {
  T e[V];
};

template <typename T>
struct vec16 {
  static constexpr int value = (sizeof(T) <= 16 && 16 % sizeof(T) == 0) ? int(16 / sizeof(T)) : 1;
};

// Programmatic dependent launch. A kernel launched with launch_dep() (launch.cuh) may be scheduled while the
// previous kernel of the stream is still draining: it waits until the predecessor has completed and its writes
// are visible, and only THEN announces that its own successor may be scheduled likewise - one level of overlap.
// (Announcing first lets a grandchild become resident while the grandparent still runs: measured on the five
// kernels of the keyed row sums with 4096 keys, that cost 110 us of 830.) Everything before the wait must stay
// off global memory. Both instructions do nothing in a kernel launched the ordinary way.
B2R_DI void grid_dep_sync()
{
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Streaming load: the matrix is read exactly once, so it bypasses L1 allocation
// (ld.global.nc.L1::no_allocate). 32-byte vectors use the 256-bit load of sm_100, which can
// also mark the line evict-first in L2. Falls back to plain loads for odd sizes.
template <typename T, int V>
B2R_DI VecOf<T, V> load_stream(const T* p)
{
  VecOf<T, V> r;
  constexpr int bytes = int(sizeof(T)) * V;
  if constexpr (bytes == 32) {
    uint32_t w[8];
    asm volatile(
      "ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
      : "l"(p));
    memcpy(&r, w, 32);
  } else if constexpr (bytes == 16) {
    uint32_t w[4];
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                 : "l"(p));
    memcpy(&r, w, 16);
  } else if constexpr (bytes == 8) {
    uint32_t w[2];
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "l"(p));
    memcpy(&r, w, 8);
  } else if constexpr (bytes == 4) {
    uint32_t a;
    // scalar loads of neighbouring lanes and passes share 32-byte sectors: let L1 keep them
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(a) : "l"(p));
    memcpy(&r, &a, 4);
  } else if constexpr (bytes == 2) {
    uint16_t a;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(a) : "l"(p));
    memcpy(&r, &a, 2);
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i)
      r.e[i] = p[i];
  }
  return r;
}

// ---------------------------------------------------------------------------------------
// Warp shuffles for any trivially copyable type, moved as 32-bit words.
// ---------------------------------------------------------------------------------------
template <typename T>
B2R_DI T shfl_xor_any(const T& v, int lane_mask)
{
  static_assert(std::is_trivially_copyable<T>::value, "accumulator must be trivially copyable");
  constexpr int words = int((sizeof(T) + 3) / 4);
  uint32_t w[words]   = {};
  memcpy(w, &v, sizeof(T));
#pragma unroll
  for (int i = 0; i < words; ++i)
    w[i] = __shfl_xor_sync(0xffffffffu, w[i], lane_mask);
  T r;
  memcpy(&r, w, sizeof(T));
  return r;
}

template <typename T>
B2R_DI T shfl_idx_any(const T& v, int src_lane)
{
  constexpr int words = int((sizeof(T) + 3) / 4);
  uint32_t w[words]   = {};
  memcpy(w, &v, sizeof(T));
#pragma unroll
  for (int i = 0; i < words; ++i)
    w[i] = __shfl_sync(0xffffffffu, w[i], src_lane);
  T r;
  memcpy(&r, w, sizeof(T));
  return r;
}

// ---------------------------------------------------------------------------------------
// Accumulator states.
//
//  * GenericState<Acc, Op>      acc = op(acc, x)            any commutative+associative op
//  * WideSumState               fp32 values summed in an fp64 accumulator (all float sums)
//  * CompensatedState<Acc>      (double sums) Kahan-Babuska-Neumaier running sum: (s, c) with the rounding
//                               error of every addition collected in c; value() = s + c.
//                               The reference compensates its add_op reductions the same way
//                               (linalg/detail/coalesced_reduction-inl.cuh:36-46), but drops
//                               the compensation when partial sums of different lanes meet;
//                               here the cross-lane / cross-warp / cross-CTA merges are
//                               compensated as well.
// ---------------------------------------------------------------------------------------
template <typename T>
B2R_DI T abs_any(T v)
{
  return v < T(0) ? -v : v;
}
template <>
B2R_DI float abs_any<float>(float v)
{
  return fabsf(v);
}
template <>
B2R_DI double abs_any<double>(double v)
{
  return fabs(v);
}

// Every state also names `carry_t`, the type in which a partial result travels between two
// kernels of one reduction (scratch memory), with carry() / push_carry().
template <typename Acc, typename Op>
struct GenericState {
  using carry_t = Acc;
  Acc v;
  B2R_DI void init(const Acc& i) { v = i; }
  B2R_DI void push(const Acc& x, Op op) { v = op(v, x); }
  B2R_DI void merge(const GenericState& o, Op op) { v = op(v, o.v); }
  B2R_DI Acc value() const { return v; }
  B2R_DI carry_t carry() const { return v; }
  B2R_DI void push_carry(const carry_t& x, Op op) { v = op(v, x); }
};

template <typename Acc>
struct CompensatedState {
  using carry_t = Acc;
  Acc s;
  Acc c;
  B2R_DI void init(const Acc& i)
  {
    s = i;
    c = Acc(0);
  }
  template <typename Op>
  B2R_DI void push(const Acc& x, Op)
  {
    const Acc t   = s + x;
    const bool ge = abs_any(s) >= abs_any(x);
    const Acc big = ge ? s : x;
    const Acc sml = ge ? x : s;
    c += (big - t) + sml;
    s = t;
  }
  template <typename Op>
  B2R_DI void merge(const CompensatedState& o, Op op)
  {
    push(o.s, op);
    c += o.c;
  }
  B2R_DI Acc value() const { return s + c; }
  B2R_DI carry_t carry() const { return s + c; }
  template <typename Op>
  B2R_DI void push_carry(const carry_t& x, Op op)
  {
    push(x, op);
  }
};

// Sum of fp32 values carried in fp64: one conversion and one double add per element instead of
// the eight fp32 operations of the compensated update, and more accurate (53-bit running sum;
// the result is rounded to fp32 once, at the very end). B200 runs fp64 adds at half the fp32
// rate, which this path - a few elements per clock per SM - does not come near.
struct WideSumState {
  using carry_t = double;
  double s;
  B2R_DI void init(const float& i) { s = double(i); }
  template <typename Op>
  B2R_DI void push(const float& x, Op)
  {
    s += double(x);
  }
  template <typename Op>
  B2R_DI void merge(const WideSumState& o, Op)
  {
    s += o.s;
  }
  B2R_DI float value() const { return float(s); }
  B2R_DI carry_t carry() const { return s; }
  template <typename Op>
  B2R_DI void push_carry(const carry_t& x, Op)
  {
    s += x;
  }
};

// Tag that operator types carry (or are mapped to) when the reduction is a plain sum and
// the accumulator is a floating-point type: selects CompensatedState.
template <typename Op>
struct is_sum_op : std::false_type {};

// float sums -> WideSumState, double sums -> CompensatedState<double>, anything else generic
template <typename Acc>
struct sum_state {
  using type = typename std::conditional<std::is_same<Acc, float>::value, WideSumState, CompensatedState<Acc>>::type;
};

template <typename Acc, typename Op>
struct state_for {
  using type = typename std::conditional<is_sum_op<Op>::value && std::is_floating_point<Acc>::value,
                                         typename sum_state<Acc>::type,
                                         GenericState<Acc, Op>>::type;
};

// ---------------------------------------------------------------------------------------
// Transposing sub-warp reduction.
//
// A group of G consecutive lanes (G a power of two, 1..32, run-time) holds U states per
// lane (U a power of two, compile-time): st[u] is this lane's partial for slot u of the
// group.  After the call the finished value of slot
//        slot(i) = prefix * n_final + i,   i in [0, n_final)
// sits in st[i] of every lane whose `writer` flag is set, where
//        m       = min(log2 G, log2 U)            halving steps
//        n_final = U >> m
//        prefix  = lane_in_group >> (log2 G - m)
//        writer  = (lane_in_group & ((1 << (log2 G - m)) - 1)) == 0
// Step k exchanges with the lane `G >> (k+1)` away; while more than one slot is left each
// lane keeps one half of its slots and hands the other half over, so the number of
// exchanges is U/2 + U/4 + ... instead of U per step.
// ---------------------------------------------------------------------------------------
template <int U, typename State, typename Op>
B2R_DI void subwarp_transpose_reduce(State (&st)[U], int lane_in_group, int G, Op op)
{
  static_assert((U & (U - 1)) == 0 && U >= 1 && U <= 32, "U must be a power of two");
#pragma unroll
  for (int k = 0; k < 5; ++k) {
    const int off = G >> (k + 1);
    if (off > 0) {
      if ((U >> k) > 1) {  // compile-time once k is unrolled
        const int n      = U >> k;
        const bool upper = (lane_in_group & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
          State keep = upper ? st[i + n / 2] : st[i];
          State give = upper ? st[i] : st[i + n / 2];
          State got  = shfl_xor_any(give, off);
          keep.merge(got, op);
          st[i] = keep;
        }
      } else {
        State got = shfl_xor_any(st[0], off);
        st[0].merge(got, op);
      }
    }
  }
}

struct SubwarpLayout {
  int n_final;  // slots finished per writer lane
  int prefix;   // first finished slot = prefix * n_final
  bool writer;
};

template <int U>
B2R_DI SubwarpLayout subwarp_layout(int lane_in_group, int G)
{
  const int lg    = 31 - __clz(G);
  constexpr int lu = ilog2_floor(U);
  const int m     = lg < lu ? lg : lu;
  SubwarpLayout l;
  l.n_final = U >> m;
  l.prefix  = lane_in_group >> (lg - m);
  l.writer  = (lane_in_group & ((1 << (lg - m)) - 1)) == 0;
  return l;
}

// Block-wide merge of one state per thread through shared memory, fixed order (warp 0
// folds the per-warp results serially), so the result does not depend on scheduling.
template <typename State, typename Op>
B2R_DI State block_merge(State st, Op op, State* smem /* >= nwarps entries */)
{
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nw   = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    State got = shfl_xor_any(st, off);
    st.merge(got, op);
  }
  if (lane == 0) smem[warp] = st;
  __syncthreads();
  if (warp == 0) {
    State r = smem[0];
    for (int w = 1; w < nw; ++w)
      r.merge(smem[w], op);
    st = r;
  }
  return st;  // valid in warp 0
}

}  // namespace detail
}  // namespace raft_b200
