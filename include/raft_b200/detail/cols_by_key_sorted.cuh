// Keyed column sums, "sort the columns, then stream tiles":
//     out[r][keys[c]] += data[r][c]          data row-major [nrows x ncols]
//
// The key of a column is the same for every row, so the columns are sorted by key ONCE per call,
// chunk by chunk (a few KB of 16-bit offsets), and the matrix is then streamed in tiles of RT rows
// x CH columns through shared memory:
//
//  cbk_sort_kernel   one CTA per chunk of CH consecutive columns: counting sort of the chunk's
//                    column offsets by key (integer shared-memory atomics) -> perm16[chunk][.] and
//                    the segment starts offs16[chunk][k].
//  cbk_tile_kernel   a CTA owns RT rows and a range of chunks. Per chunk it stages the RT x CH
//                    tile with coalesced 16-byte loads (the next tile is already in registers
//                    while the current one is consumed), then thread (r, k) adds up the tile
//                    elements of row r whose column has key k - a gather in SHARED memory, fp64
//                    running sum - into its own cell of a [RT x nkeys] table. No floating-point
//                    atomics; the only order that can vary between runs is that of the columns of
//                    one key inside a chunk (integer-atomic ranks), which the fp64 sum hides below
//                    the rounding of the result.
//  cbk_merge_kernel  when the columns of a row are split over several CTAs (few rows): folds the
//                    per-CTA tables in a fixed order.
//
// Every matrix element is read from HBM once; the extra traffic is the 2-byte offsets and segment
// starts per (row tile, chunk), which stay in L2.
#pragma once

#include "col_reduce_tma.cuh"
#include "common.cuh"
#include "launch.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kCbkTpb      = 256;
constexpr int kCbkMaxKeys  = 8192;   // [RT x nkeys] fp64 table with RT >= 1 within 64 KB
constexpr int kCbkTileBytes = 32768;  // one staged tile (RT x CH elements)
constexpr int kCbkMaxRT     = 8;      // rows per tile at most
constexpr int kCbkPad       = 4;      // tile row stride = CH + 4 elements: rows start 16-byte aligned and
                                      // the lanes of one key (8 consecutive rows) hit different banks

// Shared-memory loads by 32-bit shared address: the gather loop below spends its time on address
// arithmetic, which stays 32-bit this way.
B2R_DI unsigned lds_u16(uint32_t addr)
{
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
B2R_DI double lds_as_double(uint32_t addr, float)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return double(v);
}
B2R_DI double lds_as_double(uint32_t addr, double)
{
  double v;
  asm volatile("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(addr));
  return v;
}

struct CbkPlan {
  int RT;            // rows per tile, a power of two, at most kCbkMaxRT
  int CH;            // columns per chunk, a power of two in [256, 4096]
  int vec;           // elements per staged vector (16 bytes, or 1)
  int n_chunks;
  int y_split;       // CTAs along the columns
  int chunks_per_cta;
  int64_t n_row_tiles;
  int64_t row_tiles_per_cta;  // TMA form: a CTA walks this many row tiles
  int offs_stride;            // entries per chunk in offs16 (nkeys + 1 rounded up to 8: 16-byte rows)
  bool tma;                   // TMA-staged ring (16-byte aligned rows) or register-staged tiles
  int stages;
  size_t acc_bytes;
  size_t smem;
  size_t off_perm, off_offs, off_part, total;
};

template <typename KeyT>
__global__ void __launch_bounds__(kCbkTpb) cbk_sort_kernel(const KeyT* __restrict__ keys,
                                                          int64_t ncols,
                                                          int nkeys,
                                                          int CH,
                                                          int offs_stride,
                                                          unsigned short* __restrict__ perm16,
                                                          unsigned short* __restrict__ offs16)
{
  grid_dep_sync();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* s_cnt = reinterpret_cast<int*>(smem_raw);  // [nkeys] counts, then scatter cursors
  __shared__ int s_warp[kCbkTpb / 32];
  __shared__ int s_total;
  const int chunk    = blockIdx.x;
  const int64_t c0   = int64_t(chunk) * CH;
  const int cw       = int(ncols - c0 < CH ? ncols - c0 : CH);
  const int tid      = threadIdx.x;
  const int lane     = tid & 31;
  const int warp     = tid >> 5;
  unsigned short* po = offs16 + size_t(chunk) * offs_stride;
  unsigned short* pp = perm16 + c0;

  for (int k = tid; k < nkeys; k += kCbkTpb)
    s_cnt[k] = 0;
  __syncthreads();
  for (int c = tid; c < cw; c += kCbkTpb) {
    const long long k = static_cast<long long>(keys[c0 + c]);
    if (k >= 0 && k < nkeys) atomicAdd(&s_cnt[int(k)], 1);  // a key outside [0, nkeys) drops its column
  }
  __syncthreads();
  // exclusive scan over the keys, kCbkTpb at a time
  int run = 0;
  for (int k0 = 0; k0 < nkeys; k0 += kCbkTpb) {
    const int k = k0 + tid;
    const int t = k < nkeys ? s_cnt[k] : 0;
    int inc     = t;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += a;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const int v = lane < kCbkTpb / 32 ? s_warp[lane] : 0;
      int wi      = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += a;
      }
      if (lane < kCbkTpb / 32) s_warp[lane] = wi - v;
      if (lane == 31) s_total = wi;
    }
    __syncthreads();
    const int first = run + s_warp[warp] + inc - t;
    if (k < nkeys) {
      po[k]    = static_cast<unsigned short>(first);
      s_cnt[k] = first;  // cursor
    }
    run += s_total;
    __syncthreads();
  }
  if (tid == 0) po[nkeys] = static_cast<unsigned short>(run);
  for (int c = tid; c < cw; c += kCbkTpb) {
    const long long k = static_cast<long long>(keys[c0 + c]);
    if (k >= 0 && k < nkeys) pp[atomicAdd(&s_cnt[int(k)], 1)] = static_cast<unsigned short>(c);
  }
}

// Shared memory of one tile CTA.
template <typename T>
struct CbkSmem {
  size_t off_acc, off_tile, off_perm, off_offs, total;
};
template <typename T>
inline CbkSmem<T> cbk_smem(int RT, int CH, int nkeys)
{
  CbkSmem<T> l;
  size_t o   = 0;
  l.off_acc  = o;
  const size_t cells = size_t(RT) * nkeys;
  o += align_up((cells < size_t(kCbkTpb) ? size_t(kCbkTpb) : cells) * sizeof(double), 16);  // replicas for few pairs
  l.off_tile = o;
  o += align_up(size_t(RT) * (CH + kCbkPad) * sizeof(T), 16);
  l.off_perm = o;
  o += align_up(size_t(CH) * sizeof(unsigned short), 16);
  l.off_offs = o;
  o += align_up(size_t(nkeys + 1) * sizeof(unsigned short), 16);
  l.total = o;
  return l;
}

// VEC = 16-byte vectors when every tile row starts on a 16-byte boundary (ncols and CH multiples
// of the vector width, aligned base), else 1. NV = vectors a thread stages per tile.
template <typename T, int VEC, int NV>
__global__ void __launch_bounds__(kCbkTpb) cbk_tile_kernel(T* __restrict__ out,
                                                          double* __restrict__ partial,
                                                          const T* __restrict__ data,
                                                          const unsigned short* __restrict__ perm16,
                                                          const unsigned short* __restrict__ offs16,
                                                          int64_t nrows,
                                                          int64_t ncols,
                                                          int nkeys,
                                                          int RT,
                                                          int CH,
                                                          int offs_stride,
                                                          int n_chunks,
                                                          int chunks_per_cta,
                                                          bool reset,
                                                          CbkSmem<T> lay)
{
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* acc          = reinterpret_cast<double*>(smem_raw + lay.off_acc);           // [RT][nkeys]
  T* tile              = reinterpret_cast<T*>(smem_raw + lay.off_tile);               // [RT][CH + pad]
  unsigned short* perm = reinterpret_cast<unsigned short*>(smem_raw + lay.off_perm);  // [CH]
  unsigned short* offs = reinterpret_cast<unsigned short*>(smem_raw + lay.off_offs);  // [nkeys + 1]

  const int tid     = threadIdx.x;
  const int64_t r0  = int64_t(blockIdx.x) * RT;
  const int rt      = int(nrows - r0 < RT ? nrows - r0 : RT);
  const int ch0     = blockIdx.y * chunks_per_cta;
  int ch1           = ch0 + chunks_per_cta;
  ch1               = ch1 < n_chunks ? ch1 : n_chunks;
  const int stride  = CH + kCbkPad;
  const int lrt     = 31 - __clz(RT);
  const int vpr     = CH / VEC;            // vectors per tile row, a power of two
  const int lvpr    = 31 - __clz(vpr);
  const int n_tvec  = RT * vpr;            // vectors per tile (NV * kCbkTpb >= n_tvec)
  const int n_pairs = RT * nkeys;
  // fewer (row, key) pairs than threads: S threads share a pair, each with its own table replica
  const int S       = n_pairs < kCbkTpb ? kCbkTpb / n_pairs : 1;
  const int n_work  = n_pairs * S;

  // this thread's (row, key) pair - the row is the same for all of its pairs - and, when S > 1,
  // its slice of the pair's segment; table cell of slice s of pair (k, r): s * n_pairs + k * RT + r
  const int my_slice = S > 1 ? tid / n_pairs : 0;
  const int my_pair  = S > 1 ? tid - my_slice * n_pairs : tid;
  const int my_r     = my_pair & (RT - 1);
  const int my_k     = my_pair >> lrt;

  for (int i = tid; i < n_work; i += kCbkTpb)
    acc[i] = 0.0;

  // stage(ch): this thread's vectors of chunk ch -> registers (zero outside the matrix)
  VecOf<T, VEC> pre[NV];
  auto fetch = [&](int ch) {
    const int64_t c0 = int64_t(ch) * CH;
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int v   = q * kCbkTpb + tid;
      const int r   = v >> lvpr;
      const int cv  = v & (vpr - 1);
      const bool ok = v < n_tvec && r < rt && c0 + int64_t(cv) * VEC < ncols;  // VEC divides ncols on the vector path
      if (ok) {
        pre[q] = load_stream<T, VEC>(data + (r0 + r) * ncols + c0 + int64_t(cv) * VEC);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          pre[q].e[e] = T(0);
      }
    }
  };
  if (ch0 < ch1) fetch(ch0);
  for (int ch = ch0; ch < ch1; ++ch) {
    const int64_t c0 = int64_t(ch) * CH;
    const int cw     = int(ncols - c0 < CH ? ncols - c0 : CH);
    __syncthreads();  // the previous tile has been consumed
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int v = q * kCbkTpb + tid;
      if (v < n_tvec) {
        const int r  = v >> lvpr;
        const int cv = v & (vpr - 1);
        *reinterpret_cast<VecOf<T, VEC>*>(tile + r * stride + cv * VEC) = pre[q];
      }
    }
    for (int i = tid; i < cw; i += kCbkTpb)
      perm[i] = perm16[c0 + i];
    for (int i = tid; i <= nkeys; i += kCbkTpb)
      offs[i] = offs16[size_t(ch) * offs_stride + i];
    if (ch + 1 < ch1) fetch(ch + 1);  // in flight while this tile is consumed
    __syncthreads();
    // thread (r, k): rows vary fastest, so the lanes of one key walk the same segment
    if (my_r < rt) {
      const T* row = tile + my_r * stride;
      auto segment_sum = [&](int j0, int j1) {
        double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
        int j = j0;
        for (; j + 4 <= j1; j += 4) {
          s0 += double(row[perm[j + 0]]);
          s1 += double(row[perm[j + 1]]);
          s2 += double(row[perm[j + 2]]);
          s3 += double(row[perm[j + 3]]);
        }
        for (; j < j1; ++j)
          s0 += double(row[perm[j]]);
        return (s0 + s1) + (s2 + s3);
      };
      if (S == 1) {
        // pairs tid, tid + 256, ...: the row stays, the key advances by 256 / RT
        for (int k = my_k; k < nkeys; k += kCbkTpb >> lrt)
          acc[(k << lrt) + my_r] += segment_sum(offs[k], offs[k + 1]);
      } else if (tid < n_work) {
        const unsigned seg0 = offs[my_k], len = offs[my_k + 1] - seg0;
        acc[tid] += segment_sum(int(seg0 + len * unsigned(my_slice) / unsigned(S)),
                                int(seg0 + len * unsigned(my_slice + 1) / unsigned(S)));
      }
    }
  }
  __syncthreads();
  // acc is [k][r] (row fastest); the output is [r][k]
  if (gridDim.y == 1) {
    for (int i = tid; i < rt * nkeys; i += kCbkTpb) {
      const int r = i / nkeys;
      const int k = i - r * nkeys;
      T* dst      = out + (r0 + r) * nkeys + k;
      double v = 0.0;
      for (int sl = 0; sl < S; ++sl)
        v += acc[sl * n_pairs + (k << lrt) + r];
      *dst = T(reset ? v : double(*dst) + v);
    }
  } else {
    double* dst = partial + (size_t(blockIdx.y) * nrows + r0) * nkeys;
    for (int i = tid; i < rt * nkeys; i += kCbkTpb) {
      const int r = i / nkeys;
      const int k = i - r * nkeys;
      double v    = 0.0;
      for (int sl = 0; sl < S; ++sl)
        v += acc[sl * n_pairs + (k << lrt) + r];
      dst[i] = v;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) cbk_merge_kernel(T* __restrict__ out,
                                                       const double* __restrict__ partial,
                                                       int64_t n_cells,
                                                       int y_split,
                                                       bool reset)
{
  grid_dep_sync();
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n_cells) return;
  double s = reset ? 0.0 : double(out[i]);
  for (int y = 0; y < y_split; ++y)
    s += partial[size_t(y) * n_cells + i];
  out[i] = T(s);
}

// ---------------------------------------------------------------------------------------------
// TMA-staged form of the tile kernel (rows of the matrix start on 16-byte boundaries): a producer
// thread streams, per (row tile, chunk), the RT row pieces, the chunk's sorted offsets and its
// segment starts into a ring of shared-memory stages with bulk asynchronous copies completing on
// an mbarrier (two CTAs per SM when the table is small); kCbkConsumers threads consume the stages as above - thread (r, k) owns its table
// cell, so the only block-wide synchronisation is at the end of a row tile. A CTA walks a range of
// row tiles x a range of chunks, which keeps the ring full across row tiles.
// Every mbarrier wait is bounded; a CTA that gives up writes NaN to its outputs.
// ---------------------------------------------------------------------------------------------
constexpr int kCbkConsumers = 512;
constexpr int kCbkTmaThreads = kCbkConsumers + 32;
constexpr int kCbkMaxStages  = 4;
constexpr int kCbkRegItems   = 4;  // (key, slice) items per warp slot whose sums stay in registers

struct CbkStage {
  size_t off_tile, off_perm, off_offs, bytes;  // inside one stage
};
template <typename T>
inline CbkStage cbk_stage(int RT, int CH, int offs_stride)
{
  CbkStage s;
  size_t o   = 0;
  s.off_tile = o;
  o += align_up(size_t(RT) * (CH + kCbkPad) * sizeof(T), 128);
  s.off_perm = o;
  o += align_up(size_t(CH) * sizeof(unsigned short), 128);
  s.off_offs = o;
  o += align_up(size_t(offs_stride) * sizeof(unsigned short), 128);
  s.bytes = o;
  return s;
}

template <typename T>
__global__ void __launch_bounds__(kCbkTmaThreads, 2) cbk_tile_tma_kernel(T* __restrict__ out,
                                                                       double* __restrict__ partial,
                                                                       const T* __restrict__ data,
                                                                       const unsigned short* __restrict__ perm16,
                                                                       const unsigned short* __restrict__ offs16,
                                                                       int64_t nrows,
                                                                       int64_t ncols,
                                                                       int nkeys,
                                                                       int RT,
                                                                       int CH,
                                                                       int offs_stride,
                                                                       int n_chunks,
                                                                       int chunks_per_cta,
                                                                       int64_t n_row_tiles,
                                                                       int64_t row_tiles_per_cta,
                                                                       int STAGES,
                                                                       bool reset,
                                                                       CbkStage lay,
                                                                       size_t acc_bytes,
                                                                       RingCtl ctl)
{
  extern __shared__ __align__(128) unsigned char smem_tma[];
  double* acc           = reinterpret_cast<double*>(smem_tma);  // [S][nkeys][RT]
  unsigned char* stages = smem_tma + acc_bytes;                 // [STAGES][lay.bytes]
  const uint32_t stages_u32 = smem_u32(stages);
  __shared__ __align__(8) uint64_t s_full[kCbkMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kCbkMaxStages];
  __shared__ int s_abort;

  const int tid       = threadIdx.x;
  const bool producer = tid >= kCbkConsumers;
  const int64_t rt0   = int64_t(blockIdx.x) * row_tiles_per_cta;
  int64_t rt1         = rt0 + row_tiles_per_cta;
  rt1                 = rt1 < n_row_tiles ? rt1 : n_row_tiles;
  const int ch0       = blockIdx.y * chunks_per_cta;
  int ch1             = ch0 + chunks_per_cta;
  ch1                 = ch1 < n_chunks ? ch1 : n_chunks;
  const int n_ch      = ch1 > ch0 ? ch1 - ch0 : 0;
  const int stride    = CH + kCbkPad;
  const int lrt       = 31 - __clz(RT);
  const int n_pairs   = RT * nkeys;
  // A warp covers RT rows x G keys x Q lanes per key segment (RT * G * Q = 32): long segments are
  // shared by Q lanes (no divergence, their sums folded by shuffles), short ones get more keys per
  // warp. With fewer keys than key slots, S slices of a segment go to different slots, each with
  // its own replica of the table.
  const int lanes_per_row = 32 >> lrt;
  int Q                   = 1;
  while (Q < lanes_per_row && Q * 16 * nkeys <= CH)  // at least 16 columns per lane and segment
    Q <<= 1;
  const int lq      = 31 - __clz(Q);
  const int G       = lanes_per_row >> lq;
  const int slots   = (kCbkConsumers / 32) * G;  // (key, slice) items in flight per CTA step
  int S = 1;  // a power of two: slices are cut with shifts
  while (S * 2 * nkeys <= slots)
    S <<= 1;
  const int ls      = 31 - __clz(S);
  const int n_items = nkeys * S;
  const int n_work  = n_pairs * S;               // table cells, replicas included

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], kCbkConsumers / 32);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dep_sync();  // the set-up above touches shared memory only
  volatile int* abort_flag = &s_abort;

  if (producer) {
    // The producer WARP: lane 0 waits for the stage and announces the bytes, then every copy of the stage is
    // issued by a lane of its own - RT row pieces, the sorted offsets, the segment starts - so a stage costs
    // the issue time of one copy instead of RT + 2 (one issuing thread was what bounded the kernel with few
    // keys: 5.1 TB/s with the consumers switched off).
    const int plane  = tid - kCbkConsumers;
    long long issued = 0;
    bool alive       = true;
    for (int64_t rti = rt0; rti < rt1 && alive; ++rti) {
      const int64_t r0 = rti * RT;
      const int rt     = int(nrows - r0 < RT ? nrows - r0 : RT);
      for (int c = 0; c < n_ch; ++c) {
        const int s          = int(issued % STAGES);
        const unsigned phase = unsigned(issued / STAGES) & 1u;
        int ok               = 1;
        if (plane == 0) ok = mbar_wait_bounded(&s_empty[s], phase ^ 1u, abort_flag, ctl.limit_ns) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          alive = false;
          break;
        }
        if (issued == ctl.skip_tile && blockIdx.x == 0 && blockIdx.y == 0) {  // test hook: never requested
          ++issued;
          continue;
        }
        const int ch       = ch0 + c;
        const int64_t c0   = int64_t(ch) * CH;
        const int cw       = int(ncols - c0 < CH ? ncols - c0 : CH);
        unsigned char* st  = stages + size_t(s) * lay.bytes;
        const unsigned rb  = unsigned(cw) * unsigned(sizeof(T));           // a multiple of 16
        const unsigned pb  = unsigned(CH) * unsigned(sizeof(unsigned short));
        const unsigned ob  = unsigned(offs_stride) * unsigned(sizeof(unsigned short));
        if (plane == 0) mbar_expect_tx(&s_full[s], rb * unsigned(rt) + pb + ob);
        __syncwarp();  // the bytes are announced before any copy can complete
        for (int r = plane; r < rt; r += 32)
          bulk_load(st + lay.off_tile + size_t(r) * stride * sizeof(T), data + (r0 + r) * ncols + c0, rb, &s_full[s]);
        if (plane == (rt & 31)) bulk_load(st + lay.off_perm, perm16 + size_t(ch) * CH, pb, &s_full[s]);
        if (plane == ((rt + 1) & 31)) bulk_load(st + lay.off_offs, offs16 + size_t(ch) * offs_stride, ob, &s_full[s]);
        ++issued;
      }
    }
    if (plane == 0) {
      if (alive) producer_wait_released(s_empty, issued, STAGES, abort_flag, ctl.limit_ns);
      if (*abort_flag != 0) {
        // drain: copies already issued must land before the CTA may exit
        const long long first = issued > STAGES ? issued - STAGES : 0;
        for (long long t = first; t < issued; ++t) {
          if (t == ctl.skip_tile && blockIdx.x == 0 && blockIdx.y == 0) continue;
          mbar_drain_bounded(&s_full[t % STAGES], unsigned(t / STAGES) & 1u, ctl.limit_ns);
        }
        ring_report_timeout(ctl);
      }
    }
  } else {
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int my_r = lane & (RT - 1);
    const int my_q = (lane >> lrt) & (Q - 1);
    const int my_g = lane >> (lrt + lq);
    const int first_item = warp * G + my_g;
    const int first_k    = S > 1 ? first_item % nkeys : first_item;
    const int first_sl   = S > 1 ? first_item / nkeys : 0;
    // up to kCbkRegItems items per warp slot (a few hundred keys at most): the lane's sums stay in
    // registers for the whole row tile; more items go through the table in shared memory per tile
    const bool in_regs = n_items <= kCbkRegItems * slots;
    double run_sum[kCbkRegItems];
#pragma unroll
    for (int ii = 0; ii < kCbkRegItems; ++ii)
      run_sum[ii] = 0.0;
    for (int i = tid; i < n_work; i += kCbkConsumers)
      acc[i] = 0.0;
    asm volatile("bar.sync 1, %0;" ::"n"(kCbkConsumers) : "memory");
    long long seq = 0;
    RingPos rp{0, 0u};
    bool dead     = false;
    for (int64_t rti = rt0; rti < rt1; ++rti) {
      const int64_t r0 = rti * RT;
      const int rt     = int(nrows - r0 < RT ? nrows - r0 : RT);
      for (int c = 0; c < n_ch; ++c, ++seq) {
        if (dead) continue;
        const int s          = rp.s;
        const unsigned phase = rp.phase;
        rp.advance(1, STAGES);
        if (!mbar_wait_bounded(&s_full[s], phase, abort_flag, ctl.limit_ns)) {
          dead = true;
          continue;
        }
        const uint32_t st   = stages_u32 + uint32_t(s) * uint32_t(lay.bytes);
        const uint32_t perm = st + uint32_t(lay.off_perm);   // u16 [CH]
        const uint32_t offs = st + uint32_t(lay.off_offs);   // u16 [nkeys + 1]
        const uint32_t row  = st + uint32_t(lay.off_tile) + uint32_t(my_r * stride) * uint32_t(sizeof(T));
        const uint32_t step = uint32_t(Q) * 2u;  // bytes between this lane's consecutive offsets
        // this lane's share of slice sl of the segment of key k in the staged tile
        auto segment_sum = [&](int k, int sl) {
          const unsigned seg0 = lds_u16(offs + 2u * unsigned(k)), len = lds_u16(offs + 2u * unsigned(k) + 2u) - seg0;
          const unsigned j0 = seg0 + ((len * unsigned(sl)) >> ls);
          const unsigned j1 = seg0 + ((len * unsigned(sl + 1)) >> ls);
          double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
          uint32_t pa       = perm + 2u * (j0 + unsigned(my_q));  // address of this lane's next offset
          const uint32_t pe = perm + 2u * j1;
          for (; pa + 3u * step < pe; pa += 4u * step) {
            const unsigned a = lds_u16(pa), b = lds_u16(pa + step), c2 = lds_u16(pa + 2u * step),
                           d = lds_u16(pa + 3u * step);
            s0 += lds_as_double(row + a * unsigned(sizeof(T)), T());
            s1 += lds_as_double(row + b * unsigned(sizeof(T)), T());
            s2 += lds_as_double(row + c2 * unsigned(sizeof(T)), T());
            s3 += lds_as_double(row + d * unsigned(sizeof(T)), T());
          }
          for (; pa < pe; pa += step)
            s0 += lds_as_double(row + lds_u16(pa) * unsigned(sizeof(T)), T());
          return (s0 + s1) + (s2 + s3);
        };
        if (in_regs) {
          if (my_r < rt) {
#pragma unroll
            for (int ii = 0; ii < kCbkRegItems; ++ii) {
              const int item = first_item + ii * slots;  // item = slice * nkeys + key; slices only for ii == 0
              if (item < n_items) run_sum[ii] += segment_sum(ii == 0 ? first_k : item, ii == 0 ? first_sl : 0);
            }
          }
        } else {
          // every lane of the warp runs the same number of steps (shuffles inside)
          for (int it0 = warp * G; it0 < n_items; it0 += slots) {
            const int item  = it0 + my_g;
            const bool live = item < n_items && my_r < rt;
            double sum      = live ? segment_sum(item, 0) : 0.0;  // more items than slots: S == 1
            for (int off = RT; off < (RT << lq); off <<= 1)
              sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (live && my_q == 0) acc[(item << lrt) + my_r] += sum;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[s]);
      }
      // end of the row tile: flush the table ([k][r] -> out [r][k]) and clear it
      if (in_regs) {
#pragma unroll
        for (int ii = 0; ii < kCbkRegItems; ++ii) {
          double v = run_sum[ii];
          for (int off = RT; off < (RT << lq); off <<= 1)
            v += __shfl_xor_sync(0xffffffffu, v, off);
          const int item = first_item + ii * slots;
          if (item < n_items && my_r < rt && my_q == 0)
            acc[(ii == 0 ? first_sl * n_pairs + (first_k << lrt) : (item << lrt)) + my_r] = v;
          run_sum[ii] = 0.0;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kCbkConsumers) : "memory");
      const bool failed = *abort_flag != 0;
      const double nan  = __longlong_as_double(0x7ff8000000000000ll);
      for (int i = tid; i < rt * nkeys; i += kCbkConsumers) {
        const int r = i / nkeys;
        const int k = i - r * nkeys;
        double v    = 0.0;
        for (int sl = 0; sl < S; ++sl)
          v += acc[sl * n_pairs + (k << lrt) + r];
        if (failed) v = nan;
        if (gridDim.y == 1) {
          T* dst = out + (r0 + r) * nkeys + k;
          *dst   = T(reset ? v : double(*dst) + v);
        } else {
          partial[(size_t(blockIdx.y) * nrows + r0) * nkeys + i] = v;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kCbkConsumers) : "memory");
      for (int i = tid; i < n_work; i += kCbkConsumers)
        acc[i] = 0.0;
      asm volatile("bar.sync 1, %0;" ::"n"(kCbkConsumers) : "memory");
    }
  }
}

template <typename T>
inline bool cols_by_key_sorted_supported(int64_t nrows, int64_t ncols, int64_t nkeys)
{
  return std::is_floating_point<T>::value && nkeys >= 1 && nkeys <= kCbkMaxKeys && nrows >= 1 && ncols >= 1 &&
         ncols <= (int64_t(1) << 40);
}

// Where the sorted tiles pay off: enough work to amortise three launches, rows long enough that
// a row tile spans several chunks (the table is flushed once per row tile), and keys few enough
// that a (row, key) pair finds several columns of its key in a chunk - with one column or less
// per pair the per-pair bookkeeping dominates and shared-memory atomics are faster. Measured on
// 1000 x 100000 fp32: 8 keys 3.8 vs 0.6 TB/s, 128 keys 3.2 vs 1.2, 2048 keys 0.7 vs 1.3; on
// 4096 x 4096 with 128 keys 1.4 vs 1.7.
// Tile geometry: RT rows (the fp64 table [RT x nkeys] within 64 KB; fewer rows when that makes a
// key's segment in a chunk at least 8 columns long) x CH columns, 32 KB per tile.
template <typename T>
inline void cbk_tile_shape(int64_t nkeys, int* rt_out, int* ch_out)
{
  const int tile_elts = kCbkTileBytes / int(sizeof(T));
  int RT              = kCbkMaxRT;
  while (RT > 1 && int64_t(RT) * nkeys * int64_t(sizeof(double)) > (int64_t(64) << 10))
    RT >>= 1;
  while (RT > 2 && nkeys * 8 > (tile_elts / RT < 4096 ? tile_elts / RT : 4096))
    RT >>= 1;
  int CH = tile_elts / RT;
  if (CH > 4096) CH = 4096;
  *rt_out = RT;
  *ch_out = CH;
}

template <typename T>
inline bool cols_by_key_sorted_preferred(int64_t nrows, int64_t ncols, int64_t nkeys)
{
  if (nrows * ncols < (int64_t(1) << 23) || ncols < 8192) return false;
  int RT, CH;
  cbk_tile_shape<T>(nkeys, &RT, &CH);
  return nkeys * 4 <= CH;
}

template <typename T>
inline CbkPlan plan_cols_by_key_sorted(const T* data, int64_t nrows, int64_t ncols, int64_t nkeys)
{
  constexpr int V16 = vec16<T>::value;
  CbkPlan p         = {};
  // no more rows per tile than there are, and chunks not much wider than the matrix
  int RT, CH;
  cbk_tile_shape<T>(nkeys, &RT, &CH);
  while (RT > 1 && RT / 2 >= nrows)
    RT >>= 1;
  p.RT = RT;
  while (CH > 256 && CH / 2 >= ncols)
    CH >>= 1;
  p.CH          = CH;
  p.vec         = (V16 > 1 && ncols % V16 == 0 && aligned16(data)) ? V16 : 1;
  p.n_chunks    = int(ceil_div<int64_t>(ncols, CH));
  p.n_row_tiles = ceil_div<int64_t>(nrows, RT);
  p.offs_stride = int(ceil_div<int64_t>(nkeys + 1, 8) * 8);
  const int sms = sm_count();
  // TMA form: one CTA per SM with a ring of stages next to the fp64 table
  const CbkStage stage = cbk_stage<T>(RT, CH, p.offs_stride);
  const size_t cells   = size_t(RT) * nkeys;
  p.acc_bytes          = align_up((cells < size_t(kCbkConsumers) ? size_t(kCbkConsumers) : cells) * sizeof(double), 128);
  // two CTAs per SM when the table is small: more warps to hide the gather's latencies
  const int ctas_per_sm = p.acc_bytes + 2 * stage.bytes <= (size_t(110) << 10) ? 2 : 1;
  int stages            = int(((size_t(220) << 10) / ctas_per_sm - p.acc_bytes) / stage.bytes);
  if (stages > kCbkMaxStages) stages = kCbkMaxStages;
  p.stages = stages;
  p.tma    = tuning().colkey_tma == 1 && p.vec > 1 && stages >= 2;
  if (p.tma) {
    p.smem = p.acc_bytes + size_t(stages) * stage.bytes;
    // the split that needs the fewest waves of (SMs) CTAs; splitting the columns costs a merge
    int64_t best_cost = 0;
    const int slots_total = sms * ctas_per_sm;
    for (int y = 1; y <= 2 * slots_total && y <= p.n_chunks; ++y) {
      const int cpc      = int(ceil_div<int64_t>(p.n_chunks, y));
      const int ys       = int(ceil_div<int64_t>(p.n_chunks, cpc));
      const int64_t per_x = p.n_row_tiles * ys > slots_total ? ceil_div<int64_t>(p.n_row_tiles * ys, slots_total) : 1;
      const int64_t rtpc  = per_x < p.n_row_tiles ? per_x : p.n_row_tiles;  // row tiles per CTA
      const int64_t gx    = ceil_div<int64_t>(p.n_row_tiles, rtpc);
      const int64_t waves = ceil_div<int64_t>(gx * ys, slots_total);
      const int64_t cost  = waves * rtpc * cpc * (ys > 1 ? 51 : 50) + (ys > 1 ? 50 : 0);
      if (best_cost == 0 || cost < best_cost) {
        best_cost           = cost;
        p.y_split           = ys;
        p.chunks_per_cta    = cpc;
        p.row_tiles_per_cta = rtpc;
      }
    }
  } else {
    p.smem = cbk_smem<T>(RT, CH, int(nkeys)).total;
    // CTAs along the columns when the row tiles alone do not fill the machine
    int per_sm = int((size_t(200) << 10) / (p.smem + 1024));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    const int64_t want = int64_t(sms) * per_sm;
    int64_t ys         = p.n_row_tiles >= want ? 1 : ceil_div<int64_t>(want, p.n_row_tiles);
    if (ys > p.n_chunks) ys = p.n_chunks;
    if (ys > 65535) ys = 65535;
    p.chunks_per_cta    = int(ceil_div<int64_t>(p.n_chunks, ys));
    p.y_split           = int(ceil_div<int64_t>(p.n_chunks, p.chunks_per_cta));
    p.row_tiles_per_cta = 1;
  }
  size_t o         = 0;
  p.off_perm       = o;
  o += align_up(size_t(p.n_chunks) * size_t(CH) * sizeof(unsigned short), 256);  // whole chunks: bulk copies
  p.off_offs = o;
  o += align_up(size_t(p.n_chunks) * size_t(p.offs_stride) * sizeof(unsigned short), 256);
  p.off_part = o;
  if (p.y_split > 1) o += align_up(size_t(p.y_split) * size_t(nrows) * size_t(nkeys) * sizeof(double), 256);
  p.total = o;
  return p;
}

template <typename T, typename KeyT>
cudaError_t launch_cols_by_key_sorted(T* out,
                                      const T* data,
                                      const KeyT* keys,
                                      int64_t nrows,
                                      int64_t ncols,
                                      int64_t nkeys,
                                      bool reset,
                                      cudaStream_t stream,
                                      Workspace ws = Workspace{})
{
  constexpr int V16 = vec16<T>::value;
  const CbkPlan p   = plan_cols_by_key_sorted<T>(data, nrows, ncols, nkeys);
  Scratch scratch(ws, p.total, stream);
  if (scratch.error() != cudaSuccess) return scratch.error();
  unsigned char* base    = static_cast<unsigned char*>(scratch.get());
  unsigned short* perm16 = reinterpret_cast<unsigned short*>(base + p.off_perm);
  unsigned short* offs16 = reinterpret_cast<unsigned short*>(base + p.off_offs);
  double* partial        = reinterpret_cast<double*>(base + p.off_part);
  const int nk           = int(nkeys);
  cudaError_t e;

  (void)launch_dep(cbk_sort_kernel<KeyT>, dim3(unsigned(p.n_chunks)), dim3(kCbkTpb), size_t(nk) * sizeof(int), stream,
                   keys, ncols, nk, p.CH, p.offs_stride, perm16, offs16);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  if (p.n_row_tiles > int64_t(0x7fffffff)) return cudaErrorInvalidValue;
  if (p.tma) {
    const CbkStage stage = cbk_stage<T>(p.RT, p.CH, p.offs_stride);
    auto kern            = cbk_tile_tma_kernel<T>;
    e = ensure_dynamic_smem(kern, size_t(p.smem));
    if (e != cudaSuccess) return e;
    const dim3 grid{unsigned(ceil_div<int64_t>(p.n_row_tiles, p.row_tiles_per_cta)), unsigned(p.y_split), 1u};
    (void)launch_dep(kern, dim3(grid), dim3(kCbkTmaThreads), p.smem, stream, out, partial, data, perm16, offs16,
                     nrows, ncols, nk, p.RT, p.CH, p.offs_stride, p.n_chunks, p.chunks_per_cta, p.n_row_tiles,
                     p.row_tiles_per_cta, p.stages, reset, stage, p.acc_bytes, ring_ctl(ws.status));
  } else {
  const CbkSmem<T> lay = cbk_smem<T>(p.RT, p.CH, nk);
  const dim3 grid{unsigned(p.n_row_tiles), unsigned(p.y_split), 1u};
#define B2R_LAUNCH_CBK(VEC_, NV_)                                                                       \
  do {                                                                                                  \
    auto kern = cbk_tile_kernel<T, VEC_, NV_>;                                                          \
    if (lay.total + 1024 > (size_t(48) << 10)) {                                                        \
      e = ensure_dynamic_smem(kern, size_t(lay.total));      \
      if (e != cudaSuccess) return e;                                                                   \
    }                                                                                                   \
    kern<<<grid, kCbkTpb, lay.total, stream>>>(out, partial, data, perm16, offs16, nrows, ncols, nk,    \
                                               p.RT, p.CH, p.offs_stride, p.n_chunks, p.chunks_per_cta,  \
                                               reset, lay);                                             \
  } while (0)
  constexpr int kTileElts = kCbkTileBytes / int(sizeof(T));
  if (p.vec > 1) {
    B2R_LAUNCH_CBK(V16, kTileElts / V16 / kCbkTpb);
  } else {
    B2R_LAUNCH_CBK(1, kTileElts / kCbkTpb);
  }
#undef B2R_LAUNCH_CBK
  }
  e = cudaGetLastError();
  if (e != cudaSuccess || p.y_split == 1) return e;
  const int64_t cells = nrows * nkeys;
  (void)launch_dep(cbk_merge_kernel<T>, dim3(unsigned(ceil_div<int64_t>(cells, 256))), dim3(256), 0, stream, out,
                   partial, cells, p.y_split, reset);
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
