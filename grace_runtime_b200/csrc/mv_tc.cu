// FC layers, non-element reduces and their adjoints of the dense network on the 5th-generation tensor cores.
//
// On chunk tensors [function][atom][channel] an operation  out[row] (+)= sum_items scale * W_item^T x[item]  is a
// grouped GEMM whose long dimension is the atoms: for an output row and a tile of 128 atoms,
//     D[128 atoms][n_out] = sum_items X_item[128 atoms][K] . W_item[K][n_out],
// with X_item a contiguous block of the source tensor.  A CTA owns up to 256 / n_out atom tiles at a time and keeps two
// sets of fp32 accumulators for them in tensor memory; for every item of the row its producer warps write the tile's
// activations as hi + lo operand images into a ring of shared-memory stages (canonical K-major layout, 8-row x 16-byte
// core matrices), the item's weight image (split on the host once) arrives by one bulk asynchronous copy, and one
// thread issues tcgen05.mma kind::tf32 M = 128, N = n_out: a b ~ a_lo b_hi + a_hi b_lo + a_hi b_hi keeps fp32-level
// accuracy.  The global loads of the next two tiles are in flight in registers while a tile is written, all items of a
// row accumulate in tensor memory, and the epilogue warps write each output row once while the next row's matrix
// instructions run.
// Same mathematics as mv_kernel (chain.cu); reference: fc_fwd / mv_batch, libgrace/include/grace/fused_cpu.h:294-356,
// GPU fc_fwd4 libgrace/include/grace/kk/fused_dense.h:441-495.
//
// Every wait on the tensor cores is bounded: a wait that runs out sets the error flag, the CTA frees its tensor memory
// and returns, and the host reports the failure.
#include "mv_tc.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>

namespace gb {

namespace {

constexpr int TM = 128;         // atoms of a tile = rows of an MMA = tensor-memory lanes
constexpr int NTH = 256;
constexpr int NW = NTH / 32;
constexpr int TMEM_COLS = 512;
constexpr int MAX_TILES = 16;   // atom tiles a CTA holds accumulators for
constexpr int MAX_TENSORS = 64;
constexpr int MAX_ITEMS = 512, MAX_ROWS = 192;    // tables of an operation staged in shared memory
constexpr long long WAIT_CYCLES = 40000000LL;    // ~20 ms: far beyond any tile, far below a watchdog

// byte offset of element (r, k) of a K-major operand tile with K columns (canonical layout, no swizzle)
__host__ __device__ inline int tile_off(int r, int k, int K) { return (r >> 3) * (K >> 2) * 128 + (k >> 2) * 128 + (r & 7) * 16 + (k & 3) * 4; }

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned) __cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long make_desc(unsigned addr, int K)
{
  const unsigned long long lbo = 128 >> 4, sbo = ((K >> 2) * 128) >> 4;
  return (unsigned long long) ((addr & 0x3ffff) >> 4) | (lbo << 16) | (sbo << 32) | (1ull << 46);
}

// fp32 accumulate, tf32 x tf32, both operands K-major, M = 128, N = n
__device__ __forceinline__ unsigned make_idesc(int n) { return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned) (n >> 3) << 17) | ((unsigned) (TM >> 4) << 24); }

__device__ __forceinline__ void mma_tf32_ss(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, bool accumulate)
{
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"((unsigned) accumulate) : "memory");
}

// hi + lo split of four activations for the 3 x tf32 product.  The tensor cores read the upper 19 bits of an fp32
// operand (sign, exponent, 10 mantissa bits) and ignore the rest, so `hi` is the value itself and lo = x - trunc(x) is
// exact in fp32; lo in turn is read truncated, which leaves a relative error of 2^-20 of x - the size of the a_lo b_lo
// term the scheme drops anyway.  Two instructions per value and none of them a conversion.
__device__ __forceinline__ void split4(float4 x, float sc, float4 &hi, float4 &lo)
{
  const float v[4] = {x.x * sc, x.y * sc, x.z * sc, x.w * sc};
  float l[4];
#pragma unroll
  for (int q = 0; q < 4; q++) l[q] = v[q] - __uint_as_float(__float_as_uint(v[q]) & 0xffffe000u);
  hi = make_float4(v[0], v[1], v[2], v[3]);
  lo = make_float4(l[0], l[1], l[2], l[3]);
}

template<int NC> __device__ __forceinline__ void tmem_ld(unsigned taddr, float (&v)[NC]);

template<> __device__ __forceinline__ void tmem_ld<32>(unsigned taddr, float (&v)[32])
{
  unsigned r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

template<> __device__ __forceinline__ void tmem_ld<16>(unsigned taddr, float (&v)[16])
{
  unsigned r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// position in the loop nest (round of tiles, output row, item of the row, tile of the round)
struct Cursor {
  int tile0, nt, row, it, i0, i1, tt;
  bool valid;
};

// Activation tile of a fill: K4 = K / 4 float4 per atom row.  A warp instruction covers 8 atom rows x 4 consecutive
// float4 (64 contiguous bytes of each row in global memory, 512 contiguous bytes = 4 core matrices in shared memory:
// no bank conflicts); the 16 x CG such units of a tile go round the producer warps.
template<int K> struct TileRegs {
  static constexpr int K4 = K / 4, CG = (K4 + 3) / 4, UNITS = 16 * CG, PER = (UNITS + NW - 1) / NW;
  float4 v[PER];
};

// Warp-specialised: warps 0-7 produce (global loads two tiles ahead in registers, tf32 hi / lo operand images of a tile
// into one of S shared-memory stages, the weight image of an item into a ring of S buffers), warp 8 issues the matrix
// instructions (one thread; nothing else runs on its critical path), warps 9-12 move finished accumulators from tensor
// memory to global memory.  Two sets of accumulators (TB tiles x n_out columns each) take turns, so the epilogue of a
// row overlaps the matrix instructions of the next.  Hand-offs are mbarriers: full[s] (256 producer arrivals) / empty[s]
// (tcgen05.commit) per stage, accfull[set] (tcgen05.commit after the last item of a row) / accempty[set] (128 epilogue
// arrivals).  A wait that runs out raises `abort`, which every other wait sees, and all roles leave together.
constexpr int NPROD = NTH, NTHREADS = NTH + 32 + 128;

template<int K, int CB, int S>
__global__ void __launch_bounds__(NTHREADS, 1) mv_tc_kernel(MVTCDev op, const TensorDev *__restrict__ Tg, int ntensors, int NA,
                                                            int na, int TB, int tmem_cols, int *error)
{
  using TR = TileRegs<K>;
  constexpr int K4 = TR::K4, UNITS = TR::UNITS, PER = TR::PER;
  constexpr int A_BYTES = TM * K * 4;    // one image (hi or lo) of an activation tile
  extern __shared__ __align__(1024) char smem[];
  __shared__ unsigned long long s_full[S], s_empty[S], s_accfull[2], s_accempty[2];
  __shared__ unsigned s_tmem;
  __shared__ int s_abort;
  __shared__ TensorDev s_T[MAX_TENSORS];
  // the operation's tables: every role walks them once per fill, so they live in shared memory
  __shared__ MVItem s_items[MAX_ITEMS];
  __shared__ int s_item_off[MAX_ROWS + 1], s_row_out[MAX_ROWS];
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int N = op.n_out;
  const int W_BYTES = N * K * 4;                         // one image of a weight matrix
  char *A_st = smem;                                     // stage s at s * 2 * A_BYTES: hi, then lo
  char *W_st = smem + (size_t) S * 2 * A_BYTES;          // buffer b at b * 2 * W_BYTES: hi, then lo
  float *tr_all = reinterpret_cast<float *>(W_st + (size_t) S * 2 * W_BYTES);    // transpose buffers of the epilogue warps
  for (int q = t; q < ntensors; q += NTHREADS) s_T[q] = Tg[q];
  for (int q = t; q <= op.nrows; q += NTHREADS) s_item_off[q] = op.item_off[q];
  for (int q = t; q < op.nrows; q += NTHREADS) s_row_out[q] = op.row_out[q];
  for (int q = t; q < op.nitems; q += NTHREADS) s_items[q] = op.items[q];
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (t == 0) {
    for (int s = 0; s < S; s++) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s_full[s])), "r"(NPROD) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_empty[s])) : "memory");
    }
    for (int s = 0; s < 2; s++) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_accfull[s])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 128;" ::"r"(smem_u32(&s_accempty[s])) : "memory");
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = s_tmem;
  const int ntiles = (na + TM - 1) / TM, per_round = gridDim.x * TB;
  volatile int *abort_flag = &s_abort;

  // bounded wait that also gives up when another role did
  auto wait = [&](unsigned long long *bar, unsigned parity) -> bool {
    const unsigned addr = smem_u32(bar);
    const long long t0 = clock64();
    for (;;) {
      unsigned ok;
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok) : "r"(addr), "r"(parity), "r"(20000u) : "memory");
      if (ok) return true;
      if (*abort_flag) return false;
      if (clock64() - t0 > WAIT_CYCLES) {
        *abort_flag = 1;
        return false;
      }
    }
  };
  auto start = [&](Cursor &c, int tile0, int row) {
    c.tile0 = tile0;
    c.row = row;
    c.valid = tile0 < ntiles && row < op.nrows;
    if (!c.valid) return;
    c.nt = min(TB, ntiles - tile0);
    c.i0 = c.it = s_item_off[row];
    c.i1 = s_item_off[row + 1];
    c.tt = 0;
  };
  auto advance = [&](Cursor &c) {
    if (++c.tt < c.nt) return;
    c.tt = 0;
    if (++c.it < c.i1) return;
    int row = c.row + gridDim.y, tile0 = c.tile0;
    if (row >= op.nrows) {
      row = blockIdx.y;
      tile0 += per_round;
    }
    start(c, tile0, row);
  };
  auto next_row = [&](Cursor &c) {    // first fill of the row after c's
    int row = c.row + gridDim.y, tile0 = c.tile0;
    if (row >= op.nrows) {
      row = blockIdx.y;
      tile0 += per_round;
    }
    start(c, tile0, row);
  };

  if (warp < NW) {
    // ---------------- producers ----------------
    auto load_tile = [&](const Cursor &c, TR &r) {
      const MVItem item = s_items[c.it];
      const TensorDev src = s_T[item.src];
      const int atom0 = (c.tile0 + c.tt) * TM, valid = min(TM, na - atom0);
      const float *base = src.p + ((size_t) item.irow * NA + atom0) * src.C;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        const int u = warp + NW * j, row = (u % 16) * 8 + (lane & 7), c4 = (u / 16) * 4 + (lane >> 3);
        r.v[j] = (u < UNITS && row < valid && c4 < K4) ? __ldg(reinterpret_cast<const float4 *>(base + (size_t) row * src.C) + c4)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    };
    Cursor cur, nxt, nxt2;
    start(cur, blockIdx.x * TB, blockIdx.y);
    TR regsA, regsB;
    if (cur.valid) load_tile(cur, regsA);
    nxt = cur;
    if (cur.valid) advance(nxt);
    if (nxt.valid) load_tile(nxt, regsB);
    int fill = 0, item_no = -1;
    bool ok = true;
#ifdef GB_TC_TIMING
    long long tp_[4] = {0, 0, 0, 0}, tq_ = clock64();
#define GB_TICK(a, i) do { const long long now_ = clock64(); a[i] += now_ - tq_; tq_ = now_; } while (0)
#else
#define GB_TICK(a, i) do {} while (0)
#endif
    // one fill: `mine` holds the tile at `cur`; after its conversion it receives the tile two fills ahead
    auto step = [&](TR &mine) {
      GB_TICK(tp_, 3);
      nxt2 = nxt;
      if (nxt.valid) advance(nxt2);
      const int s = fill % S;
      // the matrix instructions that read this stage S fills ago (and everything issued before them) are done
      if (fill >= S) {
        ok = wait(&s_empty[s], (unsigned) ((fill / S - 1) & 1));
        if (!ok) return;
      }
      GB_TICK(tp_, 0);
      const MVItem item = s_items[cur.it];
      if (cur.tt == 0) {    // first tile of an item: its weight image (hi + lo, byte for byte the operand layout)
        item_no++;
        if (t == 0) {
          // one bulk asynchronous copy; its bytes are counted by this stage's `full` barrier, so the matrix instructions
          // of the fill start when the image and the 256 arrivals are there, and no producer waits for the copy
          const unsigned bar = smem_u32(&s_full[s]), dst = smem_u32(W_st + (size_t) (item_no % S) * 2 * W_BYTES);
          const char *src = op.images + (size_t) item.mat * 2 * W_BYTES;
          asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"((unsigned) (2 * W_BYTES)) : "memory");
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(dst), "l"(src), "r"((unsigned) (2 * W_BYTES)), "r"(bar) : "memory");
        }
      }
      {    // registers -> tf32 hi / lo operand images of stage s
        char *hi = A_st + (size_t) s * 2 * A_BYTES, *lo = hi + A_BYTES;
#pragma unroll
        for (int j = 0; j < PER; j++) {
          const int u = warp + NW * j, c4 = (u / 16) * 4 + (lane >> 3);
          if (u < UNITS && c4 < K4) {
            const int off = ((u % 16) * K4 + c4) * 128 + (lane & 7) * 16;
            float4 h, l;
            split4(mine.v[j], item.scale, h, l);
            *reinterpret_cast<float4 *>(hi + off) = h;
            *reinterpret_cast<float4 *>(lo + off) = l;
          }
        }
      }
      GB_TICK(tp_, 1);
      if (nxt2.valid) load_tile(nxt2, mine);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&s_full[s])) : "memory");
      GB_TICK(tp_, 2);
      fill++;
      cur = nxt;
      nxt = nxt2;
    };
    while (cur.valid && ok) {
      step(regsA);
      if (!cur.valid || !ok) break;
      step(regsB);
    }
#ifdef GB_TC_TIMING
    if (t == 0 && blockIdx.x == 1 && blockIdx.y == 0)
      printf("mv_tc K %d N %d S %d TB %d fills %d producer: wait-empty %lld W+convert %lld loads+arrive %lld other %lld\n", K, N, S, TB, fill,
             tp_[0], tp_[1], tp_[2], tp_[3]);
#endif
  } else if (warp == NW) {
    // ---------------- matrix-instruction issuer ----------------
    if (lane == 0) {
      const unsigned idesc = make_idesc(N);
      Cursor cur;
      start(cur, blockIdx.x * TB, blockIdx.y);
      int fill = 0, item_no = -1, rowc = 0;
      bool ok = true;
#ifdef GB_TC_TIMING
      long long tm_[4] = {0, 0, 0, 0}, tq_ = clock64();
#endif
      while (cur.valid && ok) {
        GB_TICK(tm_, 3);
        const int s = fill % S, set = rowc & 1;
        if (cur.tt == 0) item_no++;
        if (cur.it == cur.i0 && cur.tt == 0 && rowc >= 2) {    // first fill of a row: its accumulators were read out
          ok = wait(&s_accempty[set], (unsigned) ((rowc / 2 - 1) & 1));
          if (!ok) break;
        }
        GB_TICK(tm_, 0);
        ok = wait(&s_full[s], (unsigned) ((fill / S) & 1));
        if (!ok) break;
        GB_TICK(tm_, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned a_hi = smem_u32(A_st + (size_t) s * 2 * A_BYTES);
        const unsigned b_hi = smem_u32(W_st + (size_t) (item_no % S) * 2 * W_BYTES);
        const unsigned long long dA[2] = {make_desc(a_hi, K), make_desc(a_hi + A_BYTES, K)};
        const unsigned long long dB[2] = {make_desc(b_hi, K), make_desc(b_hi + W_BYTES, K)};
        const unsigned d = tmem + (unsigned) ((set * TB + cur.tt) * N);
        const bool acc0 = cur.it != cur.i0;
#pragma unroll
        for (int pass = 0; pass < 3; pass++) {    // small terms first: a_lo b_hi, a_hi b_lo, a_hi b_hi
          const unsigned long long a = dA[pass == 0 ? 1 : 0], b = dB[pass == 1 ? 1 : 0];
#pragma unroll
          for (int ks = 0; ks < K / 8; ks++)
            mma_tf32_ss(d, a + (unsigned long long) (ks * 16), b + (unsigned long long) (ks * 16), idesc, acc0 || pass > 0 || ks > 0);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s_empty[s])) : "memory");
        Cursor nx = cur;
        advance(nx);
        if (!nx.valid || nx.row != cur.row || nx.tile0 != cur.tile0) {    // the row is complete once these are done
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s_accfull[set])) : "memory");
          rowc++;
        }
        fill++;
        cur = nx;
        GB_TICK(tm_, 2);
      }
#ifdef GB_TC_TIMING
      if (blockIdx.x == 1 && blockIdx.y == 0)
        printf("mv_tc K %d N %d issuer: wait-accempty %lld wait-full %lld issue %lld other %lld\n", K, N, tm_[0], tm_[1], tm_[2], tm_[3]);
#endif
    }
  } else {
    // ---------------- epilogue: tensor memory -> global, once per output row ----------------
    // Each warp moves blocks of 32 atoms x CB columns of its tensor-memory lanes: registers (a lane holds one atom's
    // columns) -> a padded transpose buffer of its own -> global memory with whole 128-byte lines per store
    const int ew = warp & 3;    // the quarter of the tensor-memory lanes this warp may read (warp id modulo 4)
    float *tr = tr_all + ew * (32 * (CB + 4));
    constexpr int LPR = CB / 4, RPI = 32 / LPR;    // lanes per atom row, atom rows per store instruction
    const TensorDev dstT = s_T[op.dst];
    Cursor cur;
    start(cur, blockIdx.x * TB, blockIdx.y);
    int rowc = 0;
    bool ok = true;
#ifdef GB_TC_TIMING
    long long te_[2] = {0, 0}, tq_ = clock64();
#endif
    while (cur.valid && ok) {
      const int set = rowc & 1;
      ok = wait(&s_accfull[set], (unsigned) ((rowc / 2) & 1));
      if (!ok) break;
      GB_TICK(te_, 0);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int orow = s_row_out[cur.row], nblk = N / CB;
      const int nb = cur.nt * nblk;
      // the old values of an accumulating operation are fetched one block ahead of the block being written
      float4 old[32 / RPI], oldn[32 / RPI];
      auto load_old = [&](int b, float4 (&o)[32 / RPI]) {
        const int tt = b / nblk, c0 = (b - tt * nblk) * CB, atom0 = (cur.tile0 + tt) * TM + ew * 32;
#pragma unroll
        for (int j = 0; j < 32 / RPI; j++) {
          const int r = j * RPI + lane / LPR, cq = lane % LPR;
          o[j] = (b < nb && atom0 + r < na) ? __ldcg(reinterpret_cast<const float4 *>(dstT.p + ((size_t) orow * NA + atom0 + r) * dstT.C + c0) + cq)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      };
      if (op.accumulate) load_old(0, oldn);
      for (int b = 0; b < nb; b++) {
        const int tt = b / nblk, c0 = (b - tt * nblk) * CB;
        float v[CB];
        tmem_ld<CB>(tmem + ((unsigned) (ew * 32) << 16) + (unsigned) ((set * TB + tt) * N + c0), v);
        __syncwarp();
#pragma unroll
        for (int q = 0; q < CB / 4; q++)
          *reinterpret_cast<float4 *>(tr + lane * (CB + 4) + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        __syncwarp();
        const int atom0 = (cur.tile0 + tt) * TM + ew * 32;
        if (op.accumulate) {
#pragma unroll
          for (int j = 0; j < 32 / RPI; j++) old[j] = oldn[j];
          load_old(b + 1, oldn);
        }
#pragma unroll
        for (int j = 0; j < 32 / RPI; j++) {
          const int r = j * RPI + lane / LPR, cq = lane % LPR;
          if (atom0 + r < na) {
            float4 w = *reinterpret_cast<const float4 *>(tr + r * (CB + 4) + 4 * cq);
            if (op.accumulate) {
              w.x += old[j].x; w.y += old[j].y; w.z += old[j].z; w.w += old[j].w;
            }
            reinterpret_cast<float4 *>(dstT.p + ((size_t) orow * NA + atom0 + r) * dstT.C + c0)[cq] = w;
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&s_accempty[set])) : "memory");
      rowc++;
      next_row(cur);
      GB_TICK(te_, 1);
    }
#ifdef GB_TC_TIMING
    if (warp == NW + 1 && lane == 0 && blockIdx.x == 1 && blockIdx.y == 0)
      printf("mv_tc K %d N %d epilogue: wait-accfull %lld work %lld rows %d\n", K, N, te_[0], te_[1], rowc);
#endif
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (t == 0 && s_abort) atomicExch(error, 1);
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// activation stages, weight ring and the transpose buffers of the four epilogue warps
size_t smem_bytes(int K, int N, int S)
{
  const size_t cb = N % 32 == 0 ? 32 : 16;
  return (size_t) S * 2 * TM * K * 4 + (size_t) S * 2 * N * K * 4 + (size_t) 4 * 32 * (cb + 4) * 4;
}

int stages_for(int K, int N) { return smem_bytes(K, N, 4) <= 200 * 1024 ? 4 : 2; }

template<int K, int CB, int S>
void launch_s(const MVTCDev &op, const TensorDev *T, int ntensors, int NA, int na, int TB, int tmem_cols, dim3 grid, int *error)
{
  const size_t smem = smem_bytes(K, op.n_out, S);
  static size_t attr = 0;
  if (smem > attr) {
    GB_CUDA(cudaFuncSetAttribute((mv_tc_kernel<K, CB, S>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    attr = smem;
  }
  GB_LAUNCH((mv_tc_kernel<K, CB, S>), grid, NTHREADS, smem, op, T, ntensors, NA, na, TB, tmem_cols, error);
}

template<int K> void launch_k(const MVTCDev &op, const TensorDev *T, int ntensors, int NA, int na, int TB, dim3 grid, int *error)
{
  int tmem_cols = 32;    // a power of two that holds two sets of accumulators of TB tiles
  while (tmem_cols < 2 * TB * op.n_out) tmem_cols *= 2;
  const bool s4 = stages_for(K, op.n_out) == 4;
  if (op.n_out % 32 == 0) {
    if (s4) launch_s<K, 32, 4>(op, T, ntensors, NA, na, TB, tmem_cols, grid, error);
    else launch_s<K, 32, 2>(op, T, ntensors, NA, na, TB, tmem_cols, grid, error);
  } else {
    if (s4) launch_s<K, 16, 4>(op, T, ntensors, NA, na, TB, tmem_cols, grid, error);
    else launch_s<K, 16, 2>(op, T, ntensors, NA, na, TB, tmem_cols, grid, error);
  }
}

}    // namespace

bool MVTensorCore::eligible(const MVOp &o, const std::vector<TensorSpec> &tensors)
{
  if (o.elem || o.items.empty() || o.row_out.empty()) return false;
  if ((int) tensors.size() > MAX_TENSORS || (int) o.items.size() > MAX_ITEMS || (int) o.row_out.size() > MAX_ROWS) return false;
  const int K = o.items[0].n_in;
  if (K != 8 && K != 16 && K != 32 && K != 64) return false;
  if (o.n_out % 16 != 0 || o.n_out < 16 || o.n_out > 256) return false;
  if (tensors[o.dst].channels % 4 != 0 || tensors[o.dst].channels < o.n_out) return false;
  for (const MVItem &it : o.items)
    if (it.n_in != K || tensors[it.src].channels % 4 != 0 || tensors[it.src].channels < K) return false;
  for (size_t r = 0; r + 1 < o.item_off.size(); r++)
    if (o.item_off[r + 1] == o.item_off[r]) return false;    // a row without items has no accumulator to write
  return smem_bytes(K, o.n_out, 2) <= 220 * 1024;
}

void MVTensorCore::setup(const MVOp &o)
{
  K_ = o.items[0].n_in;
  const int N = o.n_out, K = K_;
  // one operand image per distinct matrix: B[n][k] = W[k][n] as tf32 hi, then lo (canonical K-major layout)
  std::map<int, int> index;
  std::vector<char> img;
  std::vector<MVItem> items = o.items;
  for (MVItem &it : items) {
    auto f = index.find(it.mat);
    if (f == index.end()) {
      const int id = (int) index.size();
      f = index.emplace(it.mat, id).first;
      std::vector<char> hi((size_t) N * K * 4, 0), lo((size_t) N * K * 4, 0);
      for (int n = 0; n < N; n++)
        for (int k = 0; k < K; k++) {
          const float w = o.W[(size_t) it.mat + (size_t) k * o.ldw + n];
          unsigned u;
          std::memcpy(&u, &w, 4);
          u = (u + 0x1000u) & 0xffffe000u;    // round to nearest tf32 (10-bit mantissa)
          float h;
          std::memcpy(&h, &u, 4);
          const float r = w - h;
          unsigned v;
          std::memcpy(&v, &r, 4);
          v = (v + 0x1000u) & 0xffffe000u;
          std::memcpy(hi.data() + tile_off(n, k, K), &u, 4);
          std::memcpy(lo.data() + tile_off(n, k, K), &v, 4);
        }
      img.insert(img.end(), hi.begin(), hi.end());
      img.insert(img.end(), lo.begin(), lo.end());
    }
    it.mat = f->second;    // image index instead of the offset in the fp32 weights
  }
  images_.set_label("engine:weights_tf32");
  items_.set_label("engine:tables");
  images_.ensure(img.size());
  GB_CUDA(cudaMemcpyAsync(images_.get(), img.data(), img.size(), cudaMemcpyHostToDevice, dev().stream));
  items_.upload(items);
  nitems_ = (int) items.size();
  GB_CUDA(cudaStreamSynchronize(dev().stream));
  ready_ = true;
}

void MVTensorCore::launch(const MVDev &d, const TensorDev *tensors, int ntensors, int NA, int na, int *error) const
{
  if (!ready_) throw DeviceError("tensor-core FC used before its set-up");
  if (d.nrows == 0 || na == 0) return;
  MVTCDev op{};
  op.row_out = d.row_out;
  op.item_off = d.item_off;
  op.items = items_.get();
  op.images = images_.get();
  op.n_out = d.n_out;
  op.nrows = d.nrows;
  op.nitems = nitems_;
  op.accumulate = d.accumulate;
  op.dst = d.dst;
  // one CTA per SM; two sets of accumulators share the 512 tensor-memory columns
  const int ntiles = (na + TM - 1) / TM, G = dev().sm_count;
  const int tb_max = std::max(1, std::min(MAX_TILES, TMEM_COLS / 2 / d.n_out));
  const int rounds = (ntiles + G * tb_max - 1) / (G * tb_max);
  const int TB = std::max(1, std::min(tb_max, (ntiles + G * rounds - 1) / (G * rounds)));
  const int gx = std::min(G, (ntiles + TB - 1) / TB);
  const int gy = std::max(1, std::min(d.nrows, G / gx));
  const dim3 grid(gx, gy);
  switch (K_) {
    case 8: launch_k<8>(op, tensors, ntensors, NA, na, TB, grid, error); break;
    case 16: launch_k<16>(op, tensors, ntensors, NA, na, TB, grid, error); break;
    case 32: launch_k<32>(op, tensors, ntensors, NA, na, TB, grid, error); break;
    case 64: launch_k<64>(op, tensors, ntensors, NA, na, TB, grid, error); break;
    default: throw DeviceError("tensor-core FC: unsupported input width");
  }
}

}    // namespace gb
