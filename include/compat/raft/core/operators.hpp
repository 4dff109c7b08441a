// Stand-alone versions of the functors of raft/core/operators.hpp that reduction calls name
// (reference: core/operators.hpp:27-310). Same type names, call signatures and results; unused
// trailing arguments (the element index) are accepted and ignored, as in the reference.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <type_traits>

#define RAFT_B200_HD __host__ __device__ __forceinline__

namespace raft {

// ---- unary -----------------------------------------------------------------------------------
struct identity_op {
  template <typename T, typename... Rest>
  constexpr RAFT_B200_HD T operator()(const T& x, Rest...) const
  {
    return x;
  }
};

struct void_op {
  template <typename... Rest>
  constexpr RAFT_B200_HD void operator()(Rest...) const
  {
  }
};

template <typename To>
struct cast_op {
  template <typename T, typename... Rest>
  constexpr RAFT_B200_HD To operator()(T x, Rest...) const
  {
    return static_cast<To>(x);
  }
};

struct key_op {
  template <typename P, typename... Rest>
  constexpr RAFT_B200_HD auto operator()(const P& p, Rest...) const
  {
    return p.key;
  }
};

struct value_op {
  template <typename P, typename... Rest>
  constexpr RAFT_B200_HD auto operator()(const P& p, Rest...) const
  {
    return p.value;
  }
};

struct sqrt_op {
  template <typename T, typename... Rest>
  RAFT_B200_HD T operator()(const T& x, Rest...) const
  {
    if constexpr (std::is_same<T, float>::value) {
      return sqrtf(x);
    } else {
      return static_cast<T>(sqrt(static_cast<double>(x)));
    }
  }
};

struct nz_op {
  template <typename T, typename... Rest>
  constexpr RAFT_B200_HD T operator()(const T& x, Rest...) const
  {
    return x != T(0) ? T(1) : T(0);
  }
};

struct abs_op {
  template <typename T, typename... Rest>
  RAFT_B200_HD T operator()(const T& x, Rest...) const
  {
    if constexpr (std::is_unsigned<T>::value) {
      return x;
    } else if constexpr (std::is_same<T, float>::value) {
      return fabsf(x);
    } else if constexpr (std::is_same<T, double>::value) {
      return fabs(x);
    } else {
      return x < T(0) ? T(-x) : x;
    }
  }
};

struct sq_op {
  template <typename T, typename... Rest>
  constexpr RAFT_B200_HD T operator()(const T& x, Rest...) const
  {
    return x * x;
  }
  template <typename... Rest>
  RAFT_B200_HD float operator()(const __half& x, Rest...) const  // a half is squared in float
  {
    const float f = __half2float(x);
    return f * f;
  }
};

// ---- binary ----------------------------------------------------------------------------------
#define RAFT_B200_BINARY(name, expr)                                 \
  struct name {                                                      \
    template <typename A, typename B>                                \
    constexpr RAFT_B200_HD auto operator()(const A& a, const B& b) const \
    {                                                                \
      return expr;                                                   \
    }                                                                \
  }
RAFT_B200_BINARY(sub_op, a - b);
RAFT_B200_BINARY(mul_op, a* b);
RAFT_B200_BINARY(div_op, a / b);
RAFT_B200_BINARY(greater_op, a > b);
RAFT_B200_BINARY(less_op, a < b);
RAFT_B200_BINARY(greater_or_equal_op, a >= b);
RAFT_B200_BINARY(less_or_equal_op, a <= b);
RAFT_B200_BINARY(equal_op, a == b);
RAFT_B200_BINARY(notequal_op, a != b);
#undef RAFT_B200_BINARY

struct add_op {
  template <typename A, typename B>
  constexpr RAFT_B200_HD auto operator()(const A& a, const B& b) const
  {
    if constexpr (std::is_same<A, __half>::value && std::is_same<B, __half>::value) {
      return __half2float(a) + __half2float(b);
    } else if constexpr (std::is_same<A, __half>::value) {
      return __half2float(a) + b;
    } else if constexpr (std::is_same<B, __half>::value) {
      return a + __half2float(b);
    } else {
      return a + b;
    }
  }
};

struct min_op {
  template <typename T>
  RAFT_B200_HD T operator()(const T& a, const T& b) const
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

struct max_op {
  template <typename T>
  RAFT_B200_HD T operator()(const T& a, const T& b) const
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

// smaller (argmin) / larger (argmax) value wins; on equal values the LOWER key wins in both
struct argmin_op {
  template <typename P>
  constexpr RAFT_B200_HD P operator()(const P& a, const P& b) const
  {
    return (b.value < a.value || (a.value == b.value && b.key < a.key)) ? b : a;
  }
};

struct argmax_op {
  template <typename P>
  constexpr RAFT_B200_HD P operator()(const P& a, const P& b) const
  {
    return (b.value > a.value || (a.value == b.value && b.key < a.key)) ? b : a;
  }
};

// ---- constants -------------------------------------------------------------------------------
template <typename S>
struct const_op {
  const S scalar;
  constexpr explicit const_op(const S& s) : scalar{s} {}
  template <typename... Args>
  constexpr RAFT_B200_HD S operator()(Args...) const
  {
    return scalar;
  }
};

// binary operator with its right-hand side fixed: plug_const_op<float, mul_op>(2.f)(x) == x * 2.f
template <typename C, typename BinaryOp>
struct plug_const_op {
  const C c;
  const BinaryOp composed_op;
  constexpr explicit plug_const_op(const C& s) : c{s}, composed_op{} {}
  constexpr plug_const_op(const C& s, BinaryOp o) : c{s}, composed_op{o} {}
  template <typename T>
  constexpr RAFT_B200_HD auto operator()(T a) const
  {
    return composed_op(a, c);
  }
};

template <typename T>
using add_const_op = plug_const_op<T, add_op>;
template <typename T>
using sub_const_op = plug_const_op<T, sub_op>;
template <typename T>
using mul_const_op = plug_const_op<T, mul_op>;
template <typename T>
using div_const_op = plug_const_op<T, div_op>;

}  // namespace raft
