// One-shot all-reduce (sum) of small per-GPU partials over peer memory: the exchange step of the
// row-sharded column and by-key reductions (64 column sums; a 1024 x 128 table of sums plus 1024
// int64 counts), in ONE kernel per GPU instead of a library collective per tensor.
//
// Every GPU owns an exchange area that its peers have mapped (CUDA IPC between processes, direct
// pointers inside one process):
//     data  [2 sets][world slots][slot bytes]      slot r of GPU g = what rank r sent to g
//     flags [2 sets][world][kPeerMaxCtas] u32      flag (r, c) of GPU g = tag of the call whose chunk c rank r delivered to g
// Call number n (0, 1, ...; the same on all ranks) uses set n & 1 and the tag `seq` = n mod (2^32 - 2) + 1, which
// is never 0 (the area starts zeroed) and never the tag of the call before. CTA c owns chunk c of the
// payload on every rank - the same split everywhere - and runs four phases without any grid-wide step:
//   push    plain 16-byte stores of the local chunk into slot `rank` of EVERY GPU's area, the own one included;
//   signal  a CTA barrier, then flag (rank, c) := seq in every GPU's area (st.release.sys, cumulative);
//   wait    until the OWN area's flags (r, c) are seq for all r - polling local memory only, bounded by
//           `limit_ns` of the global timer: a CTA that gives up records B2R peer status 1 and leaves its
//           chunk of the output untouched;
//   sum     the world slots of the chunk in rank order (every GPU gets the same bits), fp32 sums scaled by
//           `scale` (the deferred final_op of a mean), int64 counts as they are, written in place.
// A rank can be at most one call ahead of a peer (its call seq + 1 completes only once every peer has
// delivered seq + 1, which a peer does after it has finished reading seq), so two sets suffice and
// nothing ever needs a reset. Nothing here uses multicast or a TMA load; peers are written, never read.
//
// Payloads of up to kPeerLLBytes (the 64 column sums) take a second form with no fence and no barrier at
// all: every 4-byte word travels with the call number in ONE 8-byte store {word, seq} (such a store arrives
// whole), into a region of its own in the area, [2 sets][world][2 x kPeerLLBytes]; the receiver polls the
// words themselves until their tag is seq. Twice the bytes, half the latency: what a flag costs is the
// system-scope release behind the data and one more NVLink round trip.
#pragma once

#include "common.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kPeerMaxWorld = 16;
constexpr int kPeerMaxCtas  = 64;
constexpr int kPeerThreads  = 256;
constexpr int kPeerLLBytes  = 8192;  // largest payload of the tagged-word form

struct PeerParams {
  unsigned char* base[kPeerMaxWorld];  // exchange area of every rank, as THIS GPU addresses it
  int world;
  int rank;
  unsigned seq;                   // tag of this call, never 0
  unsigned set;                   // 0 / 1: which half of the area this call uses
  unsigned long long slot_bytes;
  unsigned long long set_stride;  // world x slot_bytes
  unsigned long long flags_off;   // byte offset of the flags
  unsigned long long ll_off;      // byte offset of the tagged-word region
  unsigned long long limit_ns;
  int* status;                    // device word of this GPU: 0 ok, 1 a wait ran out
};

B2R_DI unsigned long long global_timer_ns()
{
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
B2R_DI void st_release_sys_u32(unsigned* p, unsigned v)
{
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
B2R_DI unsigned ld_acquire_sys_u32(const unsigned* p)
{
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
B2R_DI uint4 ld_cg_u128(const void* p)
{
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Payload = [n_f32 floats | zero padding to 16 bytes][n_i64 int64 | padding]. Vector v (16 bytes) of it.
B2R_DI uint4 peer_load_local(const float* sums, int64_t n_f32, const long long* counts, int64_t n_i64, int64_t nv_f32,
                             int64_t v)
{
  uint4 r = make_uint4(0u, 0u, 0u, 0u);
  if (v < nv_f32) {
    const int64_t e = v * 4;
    if (e + 4 <= n_f32 && (reinterpret_cast<uintptr_t>(sums) & 15u) == 0) {
      r = *reinterpret_cast<const uint4*>(sums + e);
    } else {
      float t[4] = {0.f, 0.f, 0.f, 0.f};
      for (int i = 0; i < 4; ++i)
        if (e + i < n_f32) t[i] = sums[e + i];
      memcpy(&r, t, 16);
    }
  } else {
    const int64_t e = (v - nv_f32) * 2;
    long long t[2]  = {0, 0};
    for (int i = 0; i < 2; ++i)
      if (e + i < n_i64) t[i] = counts[e + i];
    memcpy(&r, t, 16);
  }
  return r;
}

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(PeerParams P,
                                                                      float* sums,
                                                                      int64_t n_f32,
                                                                      long long* counts,
                                                                      int64_t n_i64,
                                                                      float scale,
                                                                      int64_t nvec,
                                                                      int64_t vec_per_cta)
{
  const int tid        = threadIdx.x;
  const int cta        = blockIdx.x;
  const int64_t nv_f32 = (n_f32 + 3) / 4;
  const int64_t v0     = int64_t(cta) * vec_per_cta;
  int64_t v1           = v0 + vec_per_cta;
  v1                   = v1 < nvec ? v1 : nvec;
  const unsigned long long set_off = (unsigned long long)P.set * P.set_stride;
  const unsigned flag_set          = P.set * unsigned(P.world) * kPeerMaxCtas;

  // push: the local chunk into slot `rank` of every area
  for (int64_t v = v0 + tid; v < v1; v += kPeerThreads) {
    const uint4 x = peer_load_local(sums, n_f32, counts, n_i64, nv_f32, v);
    for (int p = 0; p < P.world; ++p)
      *reinterpret_cast<uint4*>(P.base[p] + set_off + (unsigned long long)P.rank * P.slot_bytes + (unsigned long long)v * 16u) = x;
  }
  // signal: the barrier orders every thread's stores before the flag writers, whose system-scope release is
  // cumulative - what this CTA stored is visible to a peer that has seen the flag
  __syncthreads();
  if (tid < P.world)
    st_release_sys_u32(reinterpret_cast<unsigned*>(P.base[tid] + P.flags_off) + flag_set + P.rank * kPeerMaxCtas + cta,
                       P.seq);
  // wait: the same chunk of every rank has arrived here (bounded)
  int ok = 1;
  if (tid < P.world) {
    const unsigned* f =
      reinterpret_cast<const unsigned*>(P.base[P.rank] + P.flags_off) + flag_set + tid * kPeerMaxCtas + cta;
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while (ld_acquire_sys_u32(f) != P.seq) {
      if ((++spins & 63u) == 0u && global_timer_ns() - t0 > P.limit_ns) {
        ok = 0;
        break;
      }
    }
  }
  ok = __syncthreads_and(ok);
  if (!ok) {
    if (tid == 0 && P.status != nullptr) atomicExch(P.status, 1);
    return;
  }
  // sum: the slots in rank order
  const unsigned char* mine = P.base[P.rank] + set_off;
  for (int64_t v = v0 + tid; v < v1; v += kPeerThreads) {
    if (v < nv_f32) {
      float a[4] = {0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < P.world; ++p) {
        const uint4 x = ld_cg_u128(mine + (unsigned long long)p * P.slot_bytes + (unsigned long long)v * 16u);
        float t[4];
        memcpy(t, &x, 16);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          a[i] += t[i];
      }
      const int64_t e = v * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (e + i < n_f32) sums[e + i] = a[i] * scale;
    } else {
      long long a[2] = {0, 0};
      for (int p = 0; p < P.world; ++p) {
        const uint4 x = ld_cg_u128(mine + (unsigned long long)p * P.slot_bytes + (unsigned long long)v * 16u);
        long long t[2];
        memcpy(t, &x, 16);
        a[0] += t[0];
        a[1] += t[1];
      }
      const int64_t e = (v - nv_f32) * 2;
      for (int i = 0; i < 2; ++i)
        if (e + i < n_i64) counts[e + i] = a[i];
    }
  }
}

// Tagged-word form: one CTA, a thread per pair of words (two floats or one int64).
__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_ll_kernel(PeerParams P,
                                                                         float* sums,
                                                                         int64_t n_f32,
                                                                         long long* counts,
                                                                         int64_t n_i64,
                                                                         float scale)
{
  const int64_t np_f32 = (n_f32 + 1) / 2;  // pairs that hold floats
  const int64_t npairs = np_f32 + n_i64;
  const unsigned long long slot = 2ull * kPeerLLBytes;
  const unsigned long long set_off = P.ll_off + (unsigned long long)P.set * slot * (unsigned long long)P.world;
  int ok = 1;
  for (int64_t i = threadIdx.x; i < npairs; i += kPeerThreads) {
    unsigned w0 = 0u, w1 = 0u;
    if (i < np_f32) {
      w0 = __float_as_uint(sums[2 * i]);
      if (2 * i + 1 < n_f32) w1 = __float_as_uint(sums[2 * i + 1]);
    } else {
      const unsigned long long c = (unsigned long long)counts[i - np_f32];
      w0 = unsigned(c);
      w1 = unsigned(c >> 32);
    }
    const uint4 x = make_uint4(w0, P.seq, w1, P.seq);
    for (int p = 0; p < P.world; ++p) {
      uint4* dst = reinterpret_cast<uint4*>(P.base[p] + set_off + (unsigned long long)P.rank * slot) + i;
      asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w)
                   : "memory");
    }
  }
  const unsigned long long t0 = global_timer_ns();
  for (int64_t i = threadIdx.x; i < npairs && ok; i += kPeerThreads) {
    float f0 = 0.f, f1 = 0.f;
    unsigned long long c = 0ull;
    for (int p = 0; p < P.world && ok; ++p) {
      const uint4* src = reinterpret_cast<const uint4*>(P.base[P.rank] + set_off + (unsigned long long)p * slot) + i;
      uint4 x;
      unsigned spins = 0;
      for (;;) {
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w) : "l"(src)
                     : "memory");
        if (x.y == P.seq && x.w == P.seq) break;
        if ((++spins & 63u) == 0u && global_timer_ns() - t0 > P.limit_ns) {
          ok = 0;
          break;
        }
      }
      f0 += __uint_as_float(x.x);
      f1 += __uint_as_float(x.z);
      c += (unsigned long long)x.x | ((unsigned long long)x.z << 32);
    }
    if (ok) {
      if (i < np_f32) {
        sums[2 * i] = f0 * scale;
        if (2 * i + 1 < n_f32) sums[2 * i + 1] = f1 * scale;
      } else {
        counts[i - np_f32] = (long long)c;
      }
    }
  }
  if (!ok && P.status != nullptr) atomicExch(P.status, 1);
}

}  // namespace detail
}  // namespace raft_b200
