// Operator vocabulary of the precompiled kernels (the set the C ABI can name), plus the
// key/value pair the argmin / argmax reductions produce.
//
// The functors follow the semantics of the reference's raft/core/operators.hpp:
//   main ops    identity_op :27-33, sq_op :93-107 (half squares in float), abs_op :85-91,
//               nz_op :77-83
//   reduce ops  add_op :109-123, min_op :167-173, max_op :175-181,
//               argmin_op :183-190, argmax_op :192-199 (both: tie -> lower key)
//   final ops   identity_op, sqrt_op :69-75, mul_const_op / div_const_op :300-310, abs_op
#pragma once

#include "common.cuh"

namespace raft_b200 {

// Same layout as raft::KeyValuePair<K, V> (core/kvp.hpp:20-27): {key, value}, no padding
// games - an array of these is what the caller's KeyValuePair array looks like in memory.
template <typename K, typename V>
struct KeyValue {
  K key;
  V value;
};

namespace op {

struct Identity {
  template <typename T, typename... I>
  B2R_HDI T operator()(const T& x, I...) const
  {
    return x;
  }
};

struct Square {
  template <typename T, typename... I>
  B2R_HDI auto operator()(const T& x, I...) const
  {
    if constexpr (std::is_same<T, __half>::value) {
      const float f = __half2float(x);
      return f * f;
    } else {
      return x * x;
    }
  }
};

struct Abs {
  template <typename T, typename... I>
  B2R_HDI auto operator()(const T& x, I...) const
  {
    if constexpr (std::is_same<T, __half>::value) {
      return fabsf(__half2float(x));
    } else if constexpr (std::is_unsigned<T>::value) {
      return x;
    } else {
      return x < T(0) ? T(-x) : x;
    }
  }
};

struct NonZero {
  template <typename T, typename... I>
  B2R_HDI auto operator()(const T& x, I...) const
  {
    if constexpr (std::is_same<T, __half>::value) {
      return __half2float(x) != 0.f ? 1.f : 0.f;
    } else {
      return x != T(0) ? T(1) : T(0);
    }
  }
};

// value -> {index along the reduced axis, value}. The reference has no public functor for
// this (its tests define one locally, cpp/tests/linalg/reduce.cu:346-349).
template <typename K>
struct ToKeyValue {
  template <typename T, typename I>
  B2R_HDI KeyValue<K, T> operator()(const T& x, I idx) const
  {
    return KeyValue<K, T>{K(idx), x};
  }
};

struct Add {
  template <typename T>
  B2R_HDI T operator()(const T& a, const T& b) const
  {
    return a + b;
  }
};

// NaN behaviour follows raft::min / raft::max for floating point (fmin / fmax: a NaN
// operand is dropped), see the reference's core/math.hpp.
struct Min {
  template <typename T>
  B2R_HDI T operator()(const T& a, const T& b) const
  {
    if constexpr (std::is_same<T, float>::value) {
      return fminf(a, b);
    } else if constexpr (std::is_same<T, double>::value) {
      return fmin(a, b);
    } else {
      return b < a ? b : a;
    }
  }
};

struct Max {
  template <typename T>
  B2R_HDI T operator()(const T& a, const T& b) const
  {
    if constexpr (std::is_same<T, float>::value) {
      return fmaxf(a, b);
    } else if constexpr (std::is_same<T, double>::value) {
      return fmax(a, b);
    } else {
      return a < b ? b : a;
    }
  }
};

struct ArgMin {
  template <typename KV>
  B2R_HDI KV operator()(const KV& a, const KV& b) const
  {
    return ((b.value < a.value) || ((a.value == b.value) && (b.key < a.key))) ? b : a;
  }
};

struct ArgMax {
  template <typename KV>
  B2R_HDI KV operator()(const KV& a, const KV& b) const
  {
    return ((b.value > a.value) || ((a.value == b.value) && (b.key < a.key))) ? b : a;
  }
};

// {key, value} -> key, converted to the index type the caller stores (raft::key_op,
// core/operators.hpp:51-57): the final op of an index-only argmin / argmax.
template <typename IndexT>
struct KeyOf {
  template <typename KV>
  B2R_HDI IndexT operator()(const KV& p) const
  {
    return IndexT(p.key);
  }
};

// Final op chosen at run time (it runs once per output, so a switch costs nothing).
struct Sqrt {
  template <typename T, typename... I>
  B2R_HDI T operator()(const T& x, I...) const
  {
    return T(sqrt(x));
  }
};

enum FinalKind : int { kFinIdentity = 0, kFinSqrt = 1, kFinMulConst = 2, kFinDivConst = 3, kFinAbs = 4 };

template <typename T>
struct RuntimeFinal {
  int kind;
  T scalar;
  B2R_HDI T operator()(const T& x) const
  {
    if constexpr (std::is_floating_point<T>::value) {
      switch (kind) {
        case kFinSqrt: return T(sqrt(x));
        case kFinMulConst: return x * scalar;
        case kFinDivConst: return x / scalar;
        case kFinAbs: return x < T(0) ? -x : x;
        default: return x;
      }
    } else if constexpr (std::is_integral<T>::value) {
      switch (kind) {
        case kFinMulConst: return x * scalar;
        case kFinDivConst: return x / scalar;
        case kFinAbs: return x < T(0) ? T(-x) : x;
        default: return x;
      }
    } else {
      return x;
    }
  }
};

}  // namespace op

namespace detail {
template <>
struct is_sum_op<op::Add> : std::true_type {};
}  // namespace detail

}  // namespace raft_b200
