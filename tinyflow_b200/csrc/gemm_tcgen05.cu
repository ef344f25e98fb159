// Tensor-core path of the dense contractions: a persistent, warp-specialised 3xFP16 GEMM on the
// Blackwell tcgen05 pipeline (TMA -> shared memory -> tcgen05.mma -> TMEM -> registers -> HBM).
//
// 3xFP16.  Every fp32 operand tensor is scaled by a power of two s chosen from its largest magnitude
// (max|a|*s in [2^14, 2^15)), and every element is split once into hi = fp16(a*s) and lo = fp16(a*s - hi)
// by a packing kernel: 22 mantissa bits, the same as a tf32 hi/lo pair, and elements down to 2^-18 of the
// tensor's maximum keep all of them (smaller ones lose absolute precision below 2^-40 of the maximum).
// The GEMM accumulates hi*hi + lo*hi + hi*lo in fp32 TMEM (the dropped lo*lo term is below 2^-22
// relative) and the epilogue multiplies by 1/(s_A*s_B), exact.  fp16 inputs run the tensor pipe at twice
// the tf32 rate and halve the operand bytes.  Packed operands are plain 2-D row-major
// matrices [rows][cols] (cols contiguous) so that one kernel serves every contraction:
//
//   matmul            A, B packed as they lie; the operand's "major" (K contiguous or M/N contiguous)
//                     is a run-time flag that only changes the TMA box shape and the UMMA descriptor.
//   conv forward      activations packed pixel-major [N * frame_h * frame_w][C] with the zero halo
//                     materialised, filters packed [Cout][tap][C]; a filter tap is then a constant
//                     row shift of the activation matrix, so the K loop is (tap, 64-channel chunk)
//                     and each step is two plain 2-D TMA boxes.  Outputs computed for halo anchors
//                     are discarded by the epilogue.
//   conv backward-data  same kernel on the packed output gradient with the flipped filter
//                     [Cin][tap'][Cout]; a strided 1x1 scatters into a zeroed dx.
//   conv backward-filter  dW[k][c][tap] = sum_rows dy[row][k] * x[row + shift(tap)][c]: both operands
//                     are M/N-major, the reduction runs over pixel rows, split over CTAs and combined
//                     with fp32 atomics.
//
// Kernel roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2-9 =
// epilogue (two per TMEM lane quarter, half the columns each).  Shared memory holds a ring of stages {A_hi, A_lo, B_hi, B_lo}
// (128-byte swizzle, 64 halves of K per stage); TMEM holds two accumulators so that promoting one group of
// stages to registers overlaps the MMAs of the next.  Every mbarrier wait is bounded: on time-out the CTA raises an
// error flag the host reads, drains its outstanding copies, frees its TMEM and returns.
#include "common.h"
#include <cuda.h>
#include <cuda_fp16.h>
#include <algorithm>
#include <mutex>
#include <type_traits>
#include <unordered_map>

namespace tf {

// ------------------------------------------------------------------------------------------------
// write versions: lets cached packs detect that their source tensor changed
// ------------------------------------------------------------------------------------------------
static std::mutex g_ver_mu;
static std::unordered_map<const void*, uint64_t> g_versions;
static uint64_t g_ver_counter = 1;
static uint64_t version_locked(const void* p) {
  auto it = g_versions.find(p);
  if (it == g_versions.end()) { g_versions[p] = ++g_ver_counter; return g_ver_counter; }
  return it->second;
}
void note_write(const void* p) {
  std::lock_guard<std::mutex> lk(g_ver_mu);
  g_versions[p] = ++g_ver_counter;
}
uint64_t version_of(const void* p) {
  std::lock_guard<std::mutex> lk(g_ver_mu);
  return version_locked(p);
}

// producer-tracked maxima: two device words per tensor, handed out from zero-filled chunks
struct AmaxSlot { uint32_t* words = nullptr; unsigned uses = 0; uint64_t version = 0; int cur = 0; };
static std::unordered_map<const void*, AmaxSlot> g_amax;
static uint32_t* g_amax_chunk = nullptr;
static int g_amax_left = 0;
AmaxOut amax_track_begin(const void* data) {
  std::lock_guard<std::mutex> lk(g_ver_mu);
  AmaxSlot& sl = g_amax[data];
  if (!sl.words) {
    if (g_amax_left < 2) {
      const int kWords = 16384;
      uint32_t* chunk = nullptr;
      if (cudaMalloc((void**)&chunk, kWords * sizeof(uint32_t)) != cudaSuccess || cudaMemset(chunk, 0, kWords * sizeof(uint32_t)) != cudaSuccess ||
          cudaDeviceSynchronize() != cudaSuccess) {
        cudaGetLastError();
        g_amax.erase(data);
        return AmaxOut{};
      }
      g_amax_chunk = chunk; g_amax_left = kWords;
    }
    sl.words = g_amax_chunk; g_amax_chunk += 2; g_amax_left -= 2;
  }
  const int k = (int)(sl.uses++ & 1u);
  sl.cur = k;
  sl.version = version_locked(data);
  return AmaxOut{sl.words + k, sl.words + (k ^ 1)};
}
const uint32_t* amax_tracked(const void* data) {
  std::lock_guard<std::mutex> lk(g_ver_mu);
  auto it = g_amax.find(data);
  if (it == g_amax.end() || !it->second.words) return nullptr;
  return it->second.version == version_locked(data) ? it->second.words + it->second.cur : nullptr;
}

// ------------------------------------------------------------------------------------------------
// device-side primitives (inline PTX)
// ------------------------------------------------------------------------------------------------
constexpr int BM = 128;            // UMMA M (TMEM lanes)
constexpr int kThreads = 320;
// The two arithmetic modes differ only in the element type of the packed operands.  A stage always holds one
// 128-byte swizzle row of K per tile row (K-major) or 128 bytes of M/N per K row (M/N-major), and is consumed by four
// MMAs; the tile byte sizes are therefore the same in both modes and only the element counts change.
enum { kArithF16 = 0, kArithTF32 = 1 };
template <int AR> struct Arith;
template <> struct Arith<kArithF16> {
  typedef __half Elem;
  static constexpr int kBK = 64;            // elements of K per stage (128 B)
  static constexpr int kGW = 64;            // M/N-major operands: elements of M/N per 128-byte group row
  static constexpr uint32_t kFormat = 0;    // instruction-descriptor operand format: f16
  // M/N-major shared-memory descriptor: 128-byte swizzle with 16-byte atoms (layout type 2), 8-row K groups 1024 B apart
  static constexpr uint32_t kMnLayout = 2, kMnSbo = 1024;
};
template <> struct Arith<kArithTF32> {
  typedef float Elem;
  static constexpr int kBK = 32;
  static constexpr int kGW = 32;
  static constexpr uint32_t kFormat = 2;    // tf32
  // 32-bit M/N-major operands exist only with the 128-byte swizzle of 32-byte atoms (layout type 1): 4-row K groups
  // 512 B apart; the tensor map of such an operand asks for the same swizzle
  static constexpr uint32_t kMnLayout = 1, kMnSbo = 512;
};
static inline int bk_of(int ar) { return ar == kArithTF32 ? 32 : 64; }
static inline int gw_of(int ar) { return ar == kArithTF32 ? 32 : 64; }
static inline int elem_of(int ar) { return ar == kArithTF32 ? 4 : 2; }
constexpr int kGroupIters = 4;     // stages accumulated in TMEM before the epilogue promotes them to registers
// A product of two data tensors (post-ReLU activations times their sparse gradients) is a sum a few large terms dominate,
// so the accumulator is as large as sum|a||b| itself and every truncating tensor-core accumulation into it costs half an
// ulp of THAT: 16 accumulations per group showed up to 16 ulp (3-4 ulp rms) on Inception-v3's filter gradients against
// 3 (0.8) for fp32 FMA.  Such launches promote after every stage (4 accumulations).  Sums with a weight operand have many
// comparable terms of both signs and stay below the fp32 FMA error at 4 stages per group.
constexpr int kGroupItersDataByData = 1;
// kind::tf32 consumes 8 elements of K per instruction, half of kind::f16's 16, and its stages hold half as many: the same
// count of truncating accumulations covers a quarter of the reduction, and the 128-channel 1x1 layers of ResNet-50 (one
// group of 16) came out at 1.05 ulp rms against 0.47 for fp32 FMA.  Two stages per group keep it under twice the FMA error.
constexpr int kGroupItersTF32 = 2;
constexpr long long kWaitCycles = 3000000000ll;   // ~1.5 s at 2 GHz: far beyond any legitimate wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises *abort_flag) if the barrier does not flip in time or another
// role already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit_cycles = kWaitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i) if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit_cycles) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// im2col-mode load over a [N][H][W][C] tensor: `pixels` consecutive base pixels starting at (w, h, n) - walking w, then h,
// then n inside the map's bounding box - each displaced by the window offset (off_w, off_h); positions outside the
// tensor read as zero.  Lands [pixels][channels of one 128-byte row], swizzled like a tiled load.
__device__ __forceinline__ void tma_load_im2col(void* dst, const CUtensorMap* map, int c, int w, int h, int n, int off_w, int off_h, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n),
                 "h"((unsigned short)off_w), "h"((unsigned short)off_h) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <int AR>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (AR == kArithF16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
  }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- CTA pairs (cta_group::2): two CTAs of a cluster on neighbouring SMs compute one 256-row tile; each loads its own 128
// rows of A and HALF of the B tile, and the tensor cores of both SMs read both halves.  All of the pair's loads report to
// the barrier of the pair's first CTA (rank 0), whose MMA warp issues for both.
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory object in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t smem_of_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_at(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tiled load into this CTA's shared memory whose bytes are counted by the barrier at `bar_cluster_addr` (any CTA of the pair)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
// arrives, once the MMAs issued so far have completed, on the barrier at this shared-memory offset in BOTH CTAs of the
// pair: one commit per CTA, each naming that CTA's barrier by its cluster address
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar) {
  const uint32_t local = smem_u32(bar);
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_of_cta(local, 0)) : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_of_cta(local, 1)) : "memory");
}
template <int AR>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (AR == kArithF16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

// Shared-memory matrix descriptor, descriptor version 1 (Blackwell), 128-byte swizzle:
//   K-major operand : rows of 128 B (64 halves / 32 floats of K), 16-byte atoms (layout type 2), 8-row groups 1024 B
//                     apart (SBO); LBO unused (= 16 B); one MMA advances the start address by 32 B.
//   MN-major operand: [K rows of one stage][128 B of M/N] per column group, column groups one stage of K rows apart
//                     (LBO).  fp16: 16-byte atoms (layout type 2), 8-row K groups 1024 B apart (SBO), one MMA (K = 16)
//                     advances the start address by 2048 B.  tf32: 32-byte atoms (layout type 1), 4-row K groups 512 B
//                     apart, one MMA (K = 8) advances it by 1024 B.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | ((uint64_t)layout_type << 61);
}

// ------------------------------------------------------------------------------------------------
// kernel parameters
// ------------------------------------------------------------------------------------------------
enum { kModeGemm = 0, kModeConv = 1, kModeWgrad = 2 };
enum { kEpiRowMajor = 0, kEpiNchw = 1, kEpiWgrad = 2 };
constexpr int kMaxTaps = 49;

struct alignas(64) GemmParams {
  CUtensorMap a_hi, a_lo, b_hi, b_lo;
  int mode, a_mn, b_mn, epi;
  int M, N;                       // valid extents of the output tile grid
  int m_tiles, n_tiles, tap_tiles;
  int k_total;                    // stages of one output tile's whole reduction
  // Schedule.  Tiles [0, full_tiles) are computed whole, round robin over the CTAs (whole waves).  The remaining
  // tail_tiles tiles - a partial wave - either run whole as well (tail_share == 0) or have their
  // tail_tiles * k_total stages cut into one contiguous range of tail_share stages per CTA, so that every SM does the
  // same amount of work; a range may cover pieces of several tiles.  Each piece leaves its raw partial sums in a
  // workspace slot and reduce_partials_kernel adds the pieces of a tile in a fixed order (no atomics: results are
  // bit-identical from run to run).
  int full_tiles, tail_tiles, tail_share, slots_per_cta;
  float* workspace;               // [slot][BN columns][128 rows] fp32
  int chunks_per_tap;             // kModeConv: K stages per tap
  int b_tap_pitch;                // kModeConv: columns per tap in the packed filter
  int ntaps;
  float* out;
  const float* a_scale; const float* b_scale;   // device words: the power-of-two scales the packs were made with
  long long ldc;                  // kEpiRowMajor
  // kEpiNchw: row m -> (image, i, j) in a frame of frame_h x frame_w, stored at output pixel
  // (oi, oj) = (i*out_sh + out_off_h, j*out_sw + out_off_w) of channel plane c: ((image*out_c + c)*out_h + oi)*out_w + oj;
  // rows with i >= valid_h, j >= valid_w or (oi, oj) outside the plane are dropped
  int frame_h, frame_w, valid_h, valid_w, out_c, out_h, out_w, out_sh, out_sw, out_off_h, out_off_w;
  int* err;                       // device-visible error word (mapped host memory)
  // im2col != 0: the activation operand A is a halo-free [N][im_h'][im_w'][C] pack read through an im2col tensor map;
  // rows of the GEMM are the im_h x im_w base pixels per image (the output positions), the map's lower corner is
  // (im_lo_w, im_lo_h) and tap t adds the window offset (tap_off[t] & 0xffff, tap_off[t] >> 16)
  int im2col, im_w, im_h, im_lo_w, im_lo_h;
  int slot, taps_per_tile;        // kModeWgrad: M-tile rows are taps_per_tile slots of `slot` input channels, one filter tap per slot
  int group_iters;                // stages accumulated in TMEM before the epilogue promotes them to registers
  int data_by_data;               // both operands are activations / gradients (filter gradients, X^T dY): host-side hint for group_iters
  // Where the two small cross terms accumulate.  0: A_lo*B_hi joins A_hi*B_hi (block 0), A_hi*B_lo alone in block 1.
  // 1: both cross terms in block 1.  2: the B stage is laid out [B_lo ; B_hi], so the wide MMA leaves A_hi*B_lo in block 0
  // and A_hi*B_hi in block 1, and A_lo*B_hi joins block 0.  In 1 and 2 the large accumulator sees one truncating
  // accumulation per K step instead of two; in 2 the narrow MMA depends on the first half of the wide one, not the last.
  int acc_layout;
  int tap_off[kMaxTaps];          // row shift per tap (applied to the activation operand A)
  short tap_col[kMaxTaps];        // first column of the tap's channels in A (space-to-depth packs keep one phase per column block)
  short tap_b[kMaxTaps];          // kModeConv: which tap block of the packed filter the tap multiplies
};

template <int BN> struct SmemLayout {
  static constexpr int kStages = BN <= 96 ? 4 : 3;
  static constexpr int kABytes = BM * 128;              // 16 KiB: 128 tile rows x one 128-byte swizzle row
  static constexpr int kBBytes = BN * 128;
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;   // + slack to align to 1024
};

// One unit of a CTA's work: `kcount` stages of tile `tile` starting at stage k0.  slot < 0: the item is the tile's
// whole reduction and its epilogue stores to the output; otherwise its partial sums go to that workspace slot.
struct WorkItem { int tile, k0, kcount, slot; };
// The sequence of items of this CTA; the three warp roles walk it independently and must see the same sequence.
struct WorkIter {
  int tile, u, u1, first_tail_tile;
  __device__ __forceinline__ explicit WorkIter(const GemmParams& p) {
    tile = blockIdx.x;
    u = u1 = first_tail_tile = 0;
    if (p.tail_share > 0) {
      u = blockIdx.x * p.tail_share;
      u1 = min(u + p.tail_share, p.tail_tiles * p.k_total);
      first_tail_tile = u / p.k_total;
    }
  }
  __device__ __forceinline__ bool next(const GemmParams& p, WorkItem& w) {
    const int whole = p.tail_share > 0 ? p.full_tiles : p.full_tiles + p.tail_tiles;
    if (tile < whole) {
      w.tile = tile; w.k0 = 0; w.kcount = p.k_total; w.slot = -1;
      tile += gridDim.x;
      return true;
    }
    if (u < u1) {
      const int t = u / p.k_total, k0 = u - t * p.k_total;
      const int len = min(p.k_total - k0, u1 - u);
      w.tile = p.full_tiles + t; w.k0 = k0; w.kcount = len;
      w.slot = blockIdx.x * p.slots_per_cta + (t - first_tail_tile);
      u += len;
      return true;
    }
    return false;
  }
};
// tile index -> coordinates; n fastest so consecutive CTAs share the A tile through L2
__device__ __forceinline__ void decode_tile(const GemmParams& p, int tile, int& mt, int& nt, int& tap) {
  nt = tile % p.n_tiles; tile /= p.n_tiles;
  tap = tile % p.tap_tiles;
  mt = tile / p.tap_tiles;
}
// Where row `row_in_tile` of tile (mt, tap) lands in the output: everything of the address but the column term.
struct RowAddr { bool ok; long long base; uint32_t col_stride; };
__device__ __forceinline__ RowAddr row_address(const GemmParams& p, int mt, int tap, int row_in_tile) {
  const long long m = (long long)mt * BM + row_in_tile;
  RowAddr r;
  r.ok = m < p.M; r.base = 0; r.col_stride = 1;
  if (p.epi == kEpiRowMajor) {
    r.base = m * p.ldc;
  } else if (p.epi == kEpiNchw) {
    const int per_img = p.frame_h * p.frame_w;
    const int img = (int)(m / per_img);
    const int rem = (int)(m - (long long)img * per_img), i = rem / p.frame_w, j = rem - i * p.frame_w;
    const int oi = i * p.out_sh + p.out_off_h, oj = j * p.out_sw + p.out_off_w;
    r.ok = r.ok && i < p.valid_h && j < p.valid_w && oi >= 0 && oi < p.out_h && oj >= 0 && oj < p.out_w;
    r.col_stride = (uint32_t)(p.out_h * p.out_w);
    r.base = ((long long)img * p.out_c) * r.col_stride + (long long)oi * p.out_w + oj;
  } else {   // kEpiWgrad: tile row -> (tap slot, input channel c), column n = output channel: out[(n * C + c) * ntaps + tap]
    const int sl = row_in_tile / p.slot, c = mt * p.slot + row_in_tile - sl * p.slot, t = tap * p.taps_per_tile + sl;
    r.ok = t < p.ntaps && c < p.M;
    r.base = (long long)c * p.ntaps + t;
    r.col_stride = (uint32_t)(p.M * p.ntaps);
  }
  return r;
}

template <int BN, int AR>
__global__ void __launch_bounds__(kThreads, 1) gemm3x_kernel(const __grid_constant__ GemmParams p) {
  using T = Arith<AR>;
  constexpr int BK = T::kBK;
  constexpr uint32_t kGroupStride = BK * 128;               // M/N-major operands: bytes between 128-byte-wide column groups
  constexpr int kTmemCols = 4 * BN <= 256 ? 256 : 512;      // two accumulators of 2*BN columns; the allocation is a power of two
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes);
  uint64_t* empty = full + L::kStages;
  uint64_t* acc_full = empty + L::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // TMEM: two accumulators of 2*BN fp32 columns each
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_sync();          // everything above (barriers, TMEM) overlapped the tail of the kernel in front; operands are read below

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool armed[L::kStages]; uint32_t armed_phase[L::kStages];
      for (int s = 0; s < L::kStages; ++s) { armed[s] = false; armed_phase[s] = 0; }
      bool ok = true;
      WorkIter iter(p);
      WorkItem w;
      while (ok && iter.next(p, w)) {
        int mt, nt, tap;
        decode_tile(p, w.tile, mt, nt, tap);
        const int m0 = mt * BM, n0 = nt * BN;
        // im2col convolution: base pixel (image, row, column) of the tile's first GEMM row
        int im_n = 0, im_y = 0, im_x = 0;
        if (p.im2col && p.mode == kModeConv) {
          const int per_img = p.im_w * p.im_h;
          im_n = m0 / per_img;
          const int rem = m0 - im_n * per_img;
          im_y = rem / p.im_w; im_x = rem - im_y * p.im_w;
        }
        for (int it = 0; it < w.kcount; ++it) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* st = smem + stage * L::kStageBytes;
          uint8_t *a_hi = st, *a_lo = st + L::kABytes;
          uint8_t *b_hi = st + 2 * L::kABytes + (p.acc_layout == 2 ? L::kBBytes : 0), *b_lo = st + 2 * L::kABytes + (p.acc_layout == 2 ? 0 : L::kBBytes);
          mbar_expect_tx(&full[stage], L::kStageBytes);
          armed[stage] = true; armed_phase[stage] = phase;
          const int git = w.k0 + it;                  // stage index within the tile's reduction
          int a_col, a_row, b_col, b_row;
          if (p.mode == kModeConv) {
            int t = git / p.chunks_per_tap, ch = git - t * p.chunks_per_tap;
            a_col = p.tap_col[t] + ch * BK; a_row = m0 + p.tap_off[t];
            b_col = p.tap_b[t] * p.b_tap_pitch + ch * BK; b_row = n0;
          } else if (p.mode == kModeWgrad) {
            int krow = git * BK;
            a_col = mt * p.slot; a_row = krow;      // per-box tap shift applied below
            b_col = n0; b_row = krow;
          } else {
            int kk = git * BK;
            if (p.a_mn) { a_col = m0; a_row = kk; } else { a_col = kk; a_row = m0; }
            if (p.b_mn) { b_col = n0; b_row = kk; } else { b_col = kk; b_row = n0; }
          }
          // M/N-major operands come through a 3-D view {group width, rows, column groups}: one copy lands
          // [groups][BK rows][128 B], the layout the M/N-major descriptor expects.
          if (p.mode == kModeConv && p.im2col) {
            const int t = git / p.chunks_per_tap;
            const int ow = p.tap_off[t] & 0xffff, oh = p.tap_off[t] >> 16;
            tma_load_im2col(a_hi, &p.a_hi, a_col, im_x + p.im_lo_w, im_y + p.im_lo_h, im_n, ow, oh, &full[stage]);
            tma_load_im2col(a_lo, &p.a_lo, a_col, im_x + p.im_lo_w, im_y + p.im_lo_h, im_n, ow, oh, &full[stage]);
          } else if (p.mode == kModeWgrad && p.im2col) {
            // the K rows of this stage are BK consecutive output pixels; every tap slot reads the input pixels they
            // touch through the im2col map, one 128-byte channel group per copy.  A slot past the last tap asks for
            // an image index beyond the batch and receives zeros.
            const int per_img = p.im_w * p.im_h;
            const int pn = a_row / per_img, prem = a_row - pn * per_img, py = prem / p.im_w, px = prem - py * p.im_w;
            const int gps = p.slot / T::kGW;
            for (int sl = 0; sl < p.taps_per_tile; ++sl) {
              const int t = tap * p.taps_per_tile + sl;
              const bool live = t < p.ntaps;
              const int ow = live ? (p.tap_off[t] & 0xffff) : 0, oh = live ? (p.tap_off[t] >> 16) : 0;
              const int bn_img = live ? pn : 0x00400000;
              for (int gq = 0; gq < gps; ++gq) {
                const int c = a_col + gq * T::kGW;
                tma_load_im2col(a_hi + (sl * gps + gq) * kGroupStride, &p.a_hi, c, px + p.im_lo_w, py + p.im_lo_h, bn_img, ow, oh, &full[stage]);
                tma_load_im2col(a_lo + (sl * gps + gq) * kGroupStride, &p.a_lo, c, px + p.im_lo_w, py + p.im_lo_h, bn_img, ow, oh, &full[stage]);
              }
            }
          } else if (p.mode == kModeWgrad) {
            // One copy per tap slot; a slot past the last tap reads rows beyond the pack (the copy still completes
            // with its full byte count and fills zeros).
            const int gps = p.slot / T::kGW;
            for (int sl = 0; sl < p.taps_per_tile; ++sl) {
              int t = tap * p.taps_per_tile + sl;
              int row = t < p.ntaps ? a_row + p.tap_off[t] : 0x40000000;
              int grp = (a_col + (t < p.ntaps ? p.tap_col[t] : 0)) / T::kGW;
              tma_load_3d(a_hi + sl * gps * kGroupStride, &p.a_hi, 0, row, grp, &full[stage]);
              tma_load_3d(a_lo + sl * gps * kGroupStride, &p.a_lo, 0, row, grp, &full[stage]);
            }
          } else if (p.a_mn) {
            tma_load_3d(a_hi, &p.a_hi, 0, a_row, a_col / T::kGW, &full[stage]);
            tma_load_3d(a_lo, &p.a_lo, 0, a_row, a_col / T::kGW, &full[stage]);
          } else {
            tma_load_2d(a_hi, &p.a_hi, a_col, a_row, &full[stage]);
            tma_load_2d(a_lo, &p.a_lo, a_col, a_row, &full[stage]);
          }
          if (p.b_mn) {
            tma_load_3d(b_hi, &p.b_hi, 0, b_row, b_col / T::kGW, &full[stage]);
            tma_load_3d(b_lo, &p.b_lo, 0, b_row, b_col / T::kGW, &full[stage]);
          } else {
            tma_load_2d(b_hi, &p.b_hi, b_col, b_row, &full[stage]);
            tma_load_2d(b_lo, &p.b_lo, b_col, b_row, &full[stage]);
          }
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag) {
        // let copies that are still in flight land before the CTA gives its shared memory back
        for (int s = 0; s < L::kStages; ++s) {
          if (!armed[s]) continue;
          long long t0 = clock64();
          while (!mbar_try_wait(&full[s], armed_phase[s]) && clock64() - t0 < 100000000ll) {}
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      // The B stage holds the two B tiles back to back ([B_lo ; B_hi] in the default accumulator layout 2), so ONE
      // instruction with N = 2*BN computes A_hi*B_lo (TMEM columns 0..BN-1) and A_hi*B_hi (columns BN..2BN-1); a second
      // one with N = BN adds A_lo*B_hi to the first block.  The two small cross terms share a block on purpose: every
      // accumulation into TMEM truncates the sum, an error proportional to the accumulator's magnitude, and the cross
      // terms are 2^-11 of the main one, so the large accumulator sees one truncation per K step instead of two.
      // instruction descriptor: D = f32 (bits 4-5 = 1), A format at bit 7, B format at bit 10, majors at bits 15 / 16,
      // N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t idesc_base = (1u << 4) | (T::kFormat << 7) | (T::kFormat << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
                                  ((uint32_t)(BM >> 4) << 24);
      const uint32_t idesc_wide = idesc_base | ((uint32_t)((2 * BN) >> 3) << 17), idesc_narrow = idesc_base | ((uint32_t)(BN >> 3) << 17);
      // K-major: one MMA advances 32 bytes along the 128-byte row; M/N-major: one MMA covers K rows of 128 bytes each
      // (16 rows of fp16, 8 of tf32), column groups kGroupStride apart
      const uint32_t a_lbo = p.a_mn ? kGroupStride : 16u, b_lbo = p.b_mn ? kGroupStride : 16u;
      const uint32_t a_kstep = p.a_mn ? kGroupStride / 4 : 32u, b_kstep = p.b_mn ? kGroupStride / 4 : 32u;
      const uint32_t a_sbo = p.a_mn ? T::kMnSbo : 1024u, b_sbo = p.b_mn ? T::kMnSbo : 1024u;
      const uint32_t a_lt = p.a_mn ? T::kMnLayout : 2u, b_lt = p.b_mn ? T::kMnLayout : 2u;
      int stage = 0; uint32_t phase = 0;
      int group = 0;            // accumulator groups issued so far (alternating TMEM buffers)
      bool ok = true;
      WorkIter iter(p);
      WorkItem w;
      while (ok && iter.next(p, w)) {
        for (int it0 = 0; it0 < w.kcount && ok; it0 += p.group_iters, ++group) {
          const int acc = group & 1;
          if (!mbar_wait(&acc_empty[acc], ((group >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + acc * 2 * BN;
          const int it1 = min(it0 + p.group_iters, w.kcount);
          for (int it = it0; it < it1; ++it) {
            if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t st = smem_u32(smem + stage * L::kStageBytes);
            const uint32_t a_hi = st, a_lo = st + L::kABytes, b_pair = st + 2 * L::kABytes;     // [B_hi ; B_lo], or [B_lo ; B_hi] in layout 2
            const uint32_t b_hi = b_pair + (p.acc_layout == 2 ? L::kBBytes : 0);
            const uint32_t d_narrow = d_tmem + (p.acc_layout == 1 ? BN : 0);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t ah = umma_desc(a_hi + k * a_kstep, a_lbo, a_sbo, a_lt), al = umma_desc(a_lo + k * a_kstep, a_lbo, a_sbo, a_lt);
              const uint64_t bw = umma_desc(b_pair + k * b_kstep, b_lbo, b_sbo, b_lt);    // N = 2*BN runs on into the second B tile
              const uint64_t bh = umma_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lt);
              umma<AR>(d_tmem, ah, bw, idesc_wide, (it > it0 || k > 0) ? 1u : 0u);
              umma<AR>(d_narrow, al, bh, idesc_narrow, 1u);
            }
            tcgen05_commit(&empty[stage]);       // frees the stage once the MMAs above have read it
            if (++stage == L::kStages) { stage = 0; phase ^= 1; }
          }
          if (ok) tcgen05_commit(&acc_full[acc]);
        }
      }
    }
  } else {
    // ===================== epilogue: warps 2..9 =====================
    // A warp may only read the TMEM lane quarter (warp % 4); two warps share each quarter and take one half of
    // the tile's columns each, so that every scheduler has two epilogue warps to alternate between (the
    // epilogue is a chain of dependent address/convert/store instructions and is issue-latency bound).
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int HC = BN / 2;                  // columns per epilogue warp
    const int row_in_tile = quarter * 32 + lane;
    const float inv_scale = (1.f / __ldg(p.a_scale)) * (1.f / __ldg(p.b_scale));     // powers of two: exact
    int group = 0;
    bool ok = true;
    WorkIter iter(p);
    WorkItem w;
    while (ok && iter.next(p, w)) {
      int mt, nt, tap;
      decode_tile(p, w.tile, mt, nt, tap);
      const int kcount = w.kcount;
      const int n0 = nt * BN + half * HC;
      const RowAddr ra = row_address(p, mt, tap, row_in_tile);
      const bool row_ok = ra.ok;
      const uint32_t col_stride = ra.col_stride;
      float* const row_out = p.out + ra.base + (long long)n0 * col_stride;
      const int ncols = max(0, min(HC, p.N - n0));
      const bool vec_ok = p.epi == kEpiRowMajor && ((ra.base + n0) & 3) == 0;

      auto wait_group = [&](int acc_buf, int grp) -> bool {   // lane 0 polls, the warp follows (keeps .sync.aligned loads converged)
        int got = lane == 0 ? (int)mbar_wait(&acc_full[acc_buf], (grp >> 1) & 1, abort_flag) : 1;
        return __shfl_sync(0xffffffffu, got, 0) != 0;
      };
      // NC values of this thread's row, columns c0.. of the warp's half; the offsets are independent of one
      // another (no serial pointer chain) and fit 32 bits (BN * plane size is far below 2^32 elements).
      auto store_cols = [&](const float* v, int c0, auto nc_tag) {
        constexpr int NC = decltype(nc_tag)::value;
        if (!row_ok || c0 >= ncols) return;
        if (vec_ok && c0 + NC <= ncols) {
          float4* dst = reinterpret_cast<float4*>(row_out + c0);
#pragma unroll
          for (int q = 0; q < NC / 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else if (c0 + NC <= ncols) {
          float* dst = row_out + (size_t)((uint32_t)c0 * col_stride);
#pragma unroll
          for (int q = 0; q < NC; ++q) dst[(size_t)((uint32_t)q * col_stride)] = v[q];
        } else {
          float* dst = row_out + (size_t)((uint32_t)c0 * col_stride);
#pragma unroll
          for (int q = 0; q < NC; ++q)
            if (c0 + q < ncols) dst[(size_t)((uint32_t)q * col_stride)] = v[q];
        }
      };

      if (w.slot < 0 && kcount <= p.group_iters) {
        // One accumulator group: stream TMEM straight to memory, 32 columns at a time.
        const int acc = group & 1;
        if (!wait_group(acc, group)) { ok = false; break; }
        ++group;
        tcgen05_fence_after();
        const uint32_t t_base = tmem_base + acc * 2 * BN + half * HC + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < HC; c0 += 32) {
          float v1[32], v2[32];
          tmem_ld32(t_base + c0, v1);
          tmem_ld32(t_base + BN + c0, v2);
          tmem_ld_wait();
          if (c0 + 32 >= HC) {     // last chunk read: the accumulator can be reused while we store
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
          }
#pragma unroll
          for (int q = 0; q < 32; ++q) v1[q] = (v1[q] + v2[q]) * inv_scale;
          store_cols(v1, c0, std::integral_constant<int, 32>{});
        }
        continue;
      }

      // The tensor core accumulates with truncation, so a long chain of MMAs into one TMEM accumulator
      // drifts; each group of group_iters stages is therefore accumulated in TMEM on its own and promoted
      // here into fp32 registers with round-to-nearest adds.
      float accv[HC];
#pragma unroll
      for (int q = 0; q < HC; ++q) accv[q] = 0.f;
      for (int it0 = 0; it0 < kcount && ok; it0 += p.group_iters, ++group) {
        const int acc = group & 1;
        if (!wait_group(acc, group)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t t_base = tmem_base + acc * 2 * BN + half * HC + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < HC; c0 += 16) {
          float v1[16], v2[16];
          tmem_ld16(t_base + c0, v1);              // the two accumulator blocks (which terms sit where: acc_layout)
          tmem_ld16(t_base + BN + c0, v2);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 16; ++q) accv[c0 + q] += v1[q] + v2[q];
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
      }
      if (!ok) break;
      if (w.slot >= 0) {
        // a piece of a split tile: raw partial sums to the workspace, [column][row] so that a warp's 32 rows coalesce
        float* ws = p.workspace + ((size_t)w.slot * BN + half * HC) * BM + row_in_tile;
#pragma unroll
        for (int q = 0; q < HC; ++q) ws[(size_t)q * BM] = accv[q];
        continue;
      }
#pragma unroll
      for (int q = 0; q < HC; ++q) accv[q] *= inv_scale;
      store_cols(accv, 0, std::integral_constant<int, HC>{});
    }
  }

  // ===================== teardown =====================
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

// ------------------------------------------------------------------------------------------------
// The same product on CTA pairs.  A cluster of two CTAs owns one 256 x 128 tile: CTA r loads rows [128 r, 128 r + 128)
// of A and rows [64 r, 64 r + 64) of the B tile (hi and lo each), so a stage is 48 KB per CTA instead of 64 KB - the
// operand traffic from L2, which is what bounds the one-CTA kernel, drops to three quarters per multiply - and four
// stages fit.  Rank 0's MMA warp issues three instructions of M = 256, N = 128 per K step for both SMs (A_hi B_hi into
// block 1; A_hi B_lo and A_lo B_hi into block 0: the N = 2 BN trick of the one-CTA kernel does not carry over, because
// a pair instruction takes the first half of its N columns from rank 0's shared memory and the second from rank 1's,
// which would interleave the blocks).  Each CTA's epilogue warps read their own 128 TMEM lanes.  K-major operands,
// whole tiles only (no split tail); every wait is bounded as in the one-CTA kernel, and both CTAs meet at a cluster
// barrier before either gives its shared memory and TMEM back.
// ------------------------------------------------------------------------------------------------
struct PairLayout {
  static constexpr int kBN = 128, kHalfN = 64, kStages = 4;
  static constexpr int kABytes = BM * 128, kBBytes = kHalfN * 128;
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;      // per CTA: 48 KiB
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;
};

template <int AR>
__global__ void __launch_bounds__(kThreads, 1) gemm3x_pair_kernel(const __grid_constant__ GemmParams p) {
  using T = Arith<AR>;
  using L = PairLayout;
  constexpr int BN = L::kBN;
  constexpr int BK = T::kBK;
  constexpr int kTmemCols = 512;                            // two accumulator sets of 2*BN fp32 columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes);      // used in rank 0 only
  uint64_t* empty = full + L::kStages;
  uint64_t* acc_full = empty + L::kStages;
  uint64_t* acc_empty = acc_full + 2;                                                    // used in rank 0 only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int pair_m_tiles = (p.m_tiles + 1) >> 1;
  const int pair_tiles = pair_m_tiles * p.n_tiles * p.tap_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 16); }    // 8 epilogue warps of each CTA
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // one warp of each CTA, same destination offset: the allocation spans both SMs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();       // the peer's barriers exist before anything is sent to them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_sync();

  auto decode = [&](int tile, int& mt, int& nt, int& tap) {
    nt = tile % p.n_tiles; tile /= p.n_tiles;
    tap = tile % p.tap_tiles;
    mt = 2 * (tile / p.tap_tiles) + (int)rank;
  };

  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = pair; ok && tile < pair_tiles; tile += npairs) {
        int mt, nt, tap;
        decode(tile, mt, nt, tap);
        const int m0 = mt * BM, n0 = nt * BN + (int)rank * L::kHalfN;
        for (int it = 0; it < p.k_total; ++it) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* st = smem + stage * L::kStageBytes;
          uint8_t *a_hi = st, *a_lo = st + L::kABytes, *b_hi = st + 2 * L::kABytes, *b_lo = b_hi + L::kBBytes;
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * L::kStageBytes);      // this CTA's bytes and the peer's
          const uint32_t bar = smem_of_cta(smem_u32(&full[stage]), 0);
          int a_col, a_row, b_col;
          if (p.mode == kModeConv) {
            const int t = it / p.chunks_per_tap, ch = it - t * p.chunks_per_tap;
            a_col = p.tap_col[t] + ch * BK; a_row = m0 + p.tap_off[t];
            b_col = p.tap_b[t] * p.b_tap_pitch + ch * BK;
          } else {
            a_col = it * BK; a_row = m0; b_col = it * BK;
          }
          tma_load_2d_pair(a_hi, &p.a_hi, a_col, a_row, bar);
          tma_load_2d_pair(a_lo, &p.a_lo, a_col, a_row, bar);
          tma_load_2d_pair(b_hi, &p.b_hi, b_col, n0, bar);
          tma_load_2d_pair(b_lo, &p.b_lo, b_col, n0, bar);
          ++issued;
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
      }
      // Rank 0's MMA warp releases stages with arrivals that are sent to both CTAs.  Stay until every stage this CTA
      // filled has been released, so that no arrival is still on its way when the CTA gives its shared memory back.
      for (int s = 0; ok && s < L::kStages && s < issued; ++s) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
        if (++stage == L::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (rank 0 for both SMs) =====================
    if (lane == 0 && rank == 0) {
      // instruction descriptor: D = f32, A / B formats, K-major both, N = BN, M = 256 (both CTAs' 128 rows)
      const uint32_t idesc = (1u << 4) | (T::kFormat << 7) | (T::kFormat << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      int stage = 0; uint32_t phase = 0;
      int group = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < pair_tiles; tile += npairs) {
        for (int it0 = 0; it0 < p.k_total && ok; it0 += p.group_iters, ++group) {
          const int acc = group & 1;
          if (!mbar_wait(&acc_empty[acc], ((group >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t d_cross = tmem_base + acc * 2 * BN, d_main = d_cross + BN;
          const int it1 = min(it0 + p.group_iters, p.k_total);
          for (int it = it0; it < it1; ++it) {
            if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t st = smem_u32(smem + stage * L::kStageBytes);
            const uint32_t a_hi = st, a_lo = st + L::kABytes, b_hi = st + 2 * L::kABytes, b_lo = b_hi + L::kBBytes;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t ah = umma_desc(a_hi + k * 32, 16, 1024, 2), al = umma_desc(a_lo + k * 32, 16, 1024, 2);
              const uint64_t bh = umma_desc(b_hi + k * 32, 16, 1024, 2), bl = umma_desc(b_lo + k * 32, 16, 1024, 2);
              const uint32_t accum = (it > it0 || k > 0) ? 1u : 0u;
              umma_pair<AR>(d_cross, ah, bl, idesc, accum);
              umma_pair<AR>(d_main, ah, bh, idesc, accum);
              umma_pair<AR>(d_cross, al, bh, idesc, 1u);
            }
            tcgen05_commit_pair(&empty[stage]);      // frees the stage in both CTAs
            if (++stage == L::kStages) { stage = 0; phase ^= 1; }
          }
          if (ok) tcgen05_commit_pair(&acc_full[acc]);
        }
      }
    }
  } else {
    // ===================== epilogue: warps 2..9 of both CTAs, each CTA its own 128 rows =====================
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int HC = BN / 2;
    const int row_in_tile = quarter * 32 + lane;
    const float inv_scale = (1.f / __ldg(p.a_scale)) * (1.f / __ldg(p.b_scale));
    const uint32_t acc_empty_rank0 = smem_of_cta(smem_u32(&acc_empty[0]), 0);      // + 8 bytes for set 1
    int group = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < pair_tiles; tile += npairs) {
      int mt, nt, tap;
      decode(tile, mt, nt, tap);
      const int n0 = nt * BN + half * HC;
      const RowAddr ra = row_address(p, mt, tap, row_in_tile);
      const bool row_ok = ra.ok && mt < p.m_tiles;
      const uint32_t col_stride = ra.col_stride;
      float* const row_out = p.out + ra.base + (long long)n0 * col_stride;
      const int ncols = max(0, min(HC, p.N - n0));
      const bool vec_ok = p.epi == kEpiRowMajor && ((ra.base + n0) & 3) == 0;
      float accv[HC];
#pragma unroll
      for (int q = 0; q < HC; ++q) accv[q] = 0.f;
      for (int it0 = 0; it0 < p.k_total && ok; it0 += p.group_iters, ++group) {
        const int acc = group & 1;
        int got = lane == 0 ? (int)mbar_wait(&acc_full[acc], (group >> 1) & 1, abort_flag) : 1;
        if (__shfl_sync(0xffffffffu, got, 0) == 0) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t t_base = tmem_base + acc * 2 * BN + half * HC + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < HC; c0 += 16) {
          float v1[16], v2[16];
          tmem_ld16(t_base + c0, v1);
          tmem_ld16(t_base + BN + c0, v2);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 16; ++q) accv[c0 + q] += v1[q] + v2[q];
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_at(acc_empty_rank0 + 8u * acc);
      }
      if (!ok) break;
      if (!row_ok) continue;
      if (vec_ok && ncols == HC) {
        float4* dst = reinterpret_cast<float4*>(row_out);
#pragma unroll
        for (int q = 0; q < HC / 4; ++q) dst[q] = make_float4(accv[4 * q] * inv_scale, accv[4 * q + 1] * inv_scale, accv[4 * q + 2] * inv_scale, accv[4 * q + 3] * inv_scale);
      } else {
#pragma unroll
        for (int q = 0; q < HC; ++q)
          if (q < ncols) row_out[(size_t)((uint32_t)q * col_stride)] = accv[q] * inv_scale;
      }
    }
  }

  // ===================== teardown =====================
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();       // neither CTA's MMAs, commits or remote arrivals are outstanding past this point
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

// Adds up the pieces of every split tile (the tail of the schedule) in a fixed order and writes the result where the
// GEMM's own epilogue would have.  grid (tail_tiles, BN / kReduceCols), block (128 rows, kReduceWays): the pieces of a
// tile are dealt round robin to the kReduceWays row groups, each adds its share in piece order, and the subtotals are
// added in row-group order - the same order every run, so the result is bit-reproducible.
constexpr int kReduceCols = 8, kReduceWays = 4;
template <int BN>
__global__ void __launch_bounds__(BM * kReduceWays) reduce_partials_kernel(const __grid_constant__ GemmParams p) {
  __shared__ float part[kReduceWays][kReduceCols][BM];
  grid_dep_sync();
  const int t = blockIdx.x;                            // tail tile
  int mt, nt, tap;
  decode_tile(p, p.full_tiles + t, mt, nt, tap);
  const int row = threadIdx.x, way = threadIdx.y;
  // CTA g of the GEMM covered stages [g * share, (g + 1) * share) of the tail; its first piece belongs to tail tile
  // (g * share) / k_total and its pieces sit in consecutive workspace slots
  const int g_first = (int)(((long long)t * p.k_total) / p.tail_share);
  const int g_last = (int)((((long long)t + 1) * p.k_total - 1) / p.tail_share);
  const int c_begin = blockIdx.y * kReduceCols;
  float sum[kReduceCols];
#pragma unroll
  for (int q = 0; q < kReduceCols; ++q) sum[q] = 0.f;
  // four pieces per trip: their loads are independent and all in flight before the first add (a tile of a long
  // reduction has dozens of pieces, and the loop would otherwise pay the memory latency once per piece)
  auto piece = [&](int g) -> const float* {
    const int slot = g * p.slots_per_cta + (t - (int)(((long long)g * p.tail_share) / p.k_total));
    return p.workspace + ((size_t)slot * BN + c_begin) * BM + row;
  };
  int g = g_first + way;
  for (; g + 3 * kReduceWays <= g_last; g += 4 * kReduceWays) {
    const float *w0 = piece(g), *w1 = piece(g + kReduceWays), *w2 = piece(g + 2 * kReduceWays), *w3 = piece(g + 3 * kReduceWays);
    float v0[kReduceCols], v1[kReduceCols], v2[kReduceCols], v3[kReduceCols];
#pragma unroll
    for (int q = 0; q < kReduceCols; ++q) { v0[q] = __ldcg(w0 + (size_t)q * BM); v1[q] = __ldcg(w1 + (size_t)q * BM); v2[q] = __ldcg(w2 + (size_t)q * BM); v3[q] = __ldcg(w3 + (size_t)q * BM); }
#pragma unroll
    for (int q = 0; q < kReduceCols; ++q) sum[q] = (((sum[q] + v0[q]) + v1[q]) + v2[q]) + v3[q];
  }
  for (; g <= g_last; g += kReduceWays) {
    const float* ws = piece(g);
#pragma unroll
    for (int q = 0; q < kReduceCols; ++q) sum[q] += __ldcg(ws + (size_t)q * BM);
  }
#pragma unroll
  for (int q = 0; q < kReduceCols; ++q) part[way][q][row] = sum[q];
  __syncthreads();
  // every row group finishes a quarter of the block's columns: subtotals added in row-group order
  const RowAddr ra = row_address(p, mt, tap, row);
  if (!ra.ok) return;
  const float inv_scale = (1.f / __ldg(p.a_scale)) * (1.f / __ldg(p.b_scale));
  constexpr int kPer = kReduceCols / kReduceWays;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int q = way * kPer + j;
    float v = part[0][q][row];
#pragma unroll
    for (int w2 = 1; w2 < kReduceWays; ++w2) v += part[w2][q][row];
    const int n = nt * BN + c_begin + q;
    if (n < p.N) p.out[ra.base + (long long)n * ra.col_stride] = v * inv_scale;
  }
}

// Exercises the bounded wait on its own: one thread waits, with a short limit, on a barrier that nothing arms; the wait
// gives up, raises the CTA's abort flag and the kernel reports it through the error word exactly as the GEMM does.
__global__ void barrier_timeout_probe_kernel(long long limit_cycles, int* err) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool flipped = mbar_wait(&bar, 0, &abort_flag, limit_cycles);
    if (!flipped && abort_flag && err) atomicExch(err, 1);
  }
}

// ------------------------------------------------------------------------------------------------
// packing kernels (fp32 -> power-of-two scale + hi / lo fp16 pair)
// ------------------------------------------------------------------------------------------------
// Largest magnitude of a tensor, as the bit pattern of a non-negative float (unsigned order = float order).
__global__ void __launch_bounds__(256) amax_kernel(const float* __restrict__ src, long long n, uint32_t* __restrict__ amax) {
  grid_dep_sync();
  uint32_t m = 0;
  const long long stride = (long long)gridDim.x * blockDim.x, tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  auto fold = [&](float4 v) {
    m = max(max(m, __float_as_uint(fabsf(v.x))), max(__float_as_uint(fabsf(v.y)), max(__float_as_uint(fabsf(v.z)), __float_as_uint(fabsf(v.w)))));
  };
  if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const float4* s4 = reinterpret_cast<const float4*>(src);
    const long long n4 = n / 4;
    long long i = tid;
    for (; i + 3 * stride < n4; i += 4 * stride) {       // four independent 16-byte loads in flight per thread
      float4 a = __ldg(s4 + i), b = __ldg(s4 + i + stride), c = __ldg(s4 + i + 2 * stride), d = __ldg(s4 + i + 3 * stride);
      fold(a); fold(b); fold(c); fold(d);
    }
    for (; i < n4; i += stride) fold(__ldg(s4 + i));
    for (long long k = n4 * 4 + tid; k < n; k += stride) m = max(m, __float_as_uint(fabsf(__ldg(src + k))));
  } else {
    for (long long i = tid; i < n; i += stride) m = max(m, __float_as_uint(fabsf(__ldg(src + i))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m) atomicMax(amax, m);
}
// Scale words of one pack: amax[0..1] alternate between uses (the pack kernel of use k reads amax[k & 1] and clears
// amax[(k + 1) & 1] for the next use, so no separate clearing launch is needed), scale = the power of two in force.
struct ScaleRef { const uint32_t* amax_cur; uint32_t* amax_next; float* scale; };
// s = 2^(14 - floor(log2 amax)): amax * s lies in [2^14, 2^15), below the fp16 maximum 65504 after rounding
__device__ __forceinline__ float scale_from_amax(uint32_t bits) {
  int e = (int)((bits >> 23) & 0xff);
  if (bits == 0 || e == 0xff) return 1.f;             // all zero, or Inf/NaN inside (the results are meaningless then)
  if (e == 0) e = 1;
  int se = 14 - (e - 127);
  se = se > 120 ? 120 : (se < -120 ? -120 : se);
  return __uint_as_float((uint32_t)(se + 127) << 23);
}
// A tf32 pack is not scaled: its ScaleRef has no amax word and the scale in force is 1.
__device__ __forceinline__ float pack_scale(const ScaleRef& r, bool first_thread) {
  const float s = r.amax_cur ? scale_from_amax(__ldg(r.amax_cur)) : 1.f;
  if (first_thread) { *r.scale = s; if (r.amax_next) *r.amax_next = 0; }
  return s;
}
// hi / lo pair of one value: fp16 (22 mantissa bits together) or tf32 (round to nearest, low 13 bits zero)
__device__ __forceinline__ void split_pair(float a, __half& hi, __half& lo) {
  hi = __float2half_rn(a);
  lo = __float2half_rn(a - __half2float(hi));
}
__device__ __forceinline__ float tf32_rn(float a) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(a));
  return __uint_as_float(r);
}
__device__ __forceinline__ void split_pair(float a, float& hi, float& lo) {
  hi = tf32_rn(a);
  lo = tf32_rn(a - hi);
}
// eight consecutive values -> eight hi and eight lo elements at hi + o, lo + o (o a multiple of 8): 16-byte stores
__device__ __forceinline__ void store8(__half* hi, __half* lo, long long o, const float* v) {
  __align__(16) __half2 h[4];
  __align__(16) __half2 l[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    h[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
    const float2 hf = __half22float2(h[e]);
    l[e] = __floats2half2_rn(v[2 * e] - hf.x, v[2 * e + 1] - hf.y);
  }
  *reinterpret_cast<uint4*>(hi + o) = *reinterpret_cast<const uint4*>(h);
  *reinterpret_cast<uint4*>(lo + o) = *reinterpret_cast<const uint4*>(l);
}
__device__ __forceinline__ void store8(float* hi, float* lo, long long o, const float* v) {
  float h[8], l[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) split_pair(v[e], h[e], l[e]);
  float4* hp = reinterpret_cast<float4*>(hi + o);
  float4* lp = reinterpret_cast<float4*>(lo + o);
  hp[0] = make_float4(h[0], h[1], h[2], h[3]); hp[1] = make_float4(h[4], h[5], h[6], h[7]);
  lp[0] = make_float4(l[0], l[1], l[2], l[3]); lp[1] = make_float4(l[4], l[5], l[6], l[7]);
}

// rows x cols row-major (pitch src_ld) -> hi/lo with pitch dst_ld.  VEC8: eight consecutive columns per thread
// (two 16-byte loads, one 16-byte store each of hi and lo); needs cols and src_ld multiples of 8 and a 16-byte
// aligned source (the packs' pitch is a multiple of 64).
template <bool VEC8, class E>
__global__ void __launch_bounds__(256) pack_matrix_kernel(const float* __restrict__ src, long long src_ld, E* __restrict__ hi, E* __restrict__ lo,
                                                          long long dst_ld, long long rows, long long cols, ScaleRef sr) {
  grid_dep_sync();
  const float sc = pack_scale(sr, blockIdx.x == 0 && threadIdx.x == 0);
  const long long stride = (long long)gridDim.x * blockDim.x;
  if (VEC8) {
    const long long cols8 = cols >> 3, total = rows * cols8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const long long r = i / cols8, c = (i - r * cols8) << 3;
      const float4 a = __ldg(reinterpret_cast<const float4*>(src + r * src_ld + c));
      const float4 b = __ldg(reinterpret_cast<const float4*>(src + r * src_ld + c) + 1);
      const float v[8] = {a.x * sc, a.y * sc, a.z * sc, a.w * sc, b.x * sc, b.y * sc, b.z * sc, b.w * sc};
      store8(hi, lo, r * dst_ld + c, v);
    }
  } else {
    const long long total = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      long long r = i / cols, c = i - r * cols;
      E h, l;
      split_pair(src[r * src_ld + c] * sc, h, l);
      hi[r * dst_ld + c] = h;
      lo[r * dst_ld + c] = l;
    }
  }
}

// NCHW activations -> pixel-major frame [N][frame_h][frame_w][pitch]:
//   dst(n, i, j, dst_c0 + c) = src(n, c, i * sh - off_h, j * sw - off_w) when that sample exists, else 0
// (off > 0 places the source behind a zero halo; off <= 0 with sh > 1 selects one phase of a strided sampling).
// Channels c < c_limit are written (zeros past C).  One block moves 32 frame columns x TC channels of one frame
// row through shared memory: reads run along w (TC/8 independent loads per thread in flight), writes along c as
// 16-byte vectors (8 halves) of hi and of lo.
struct PackGeom { int N, C, H, W, frame_h, frame_w, off_h, off_w, sh, sw, pitch, dst_c0, c_limit; };
// RELU: the source is the input of a ReLU; the kernel applies it, writes the fp32 result to y_out (same layout as the
// source), records max|y| like the stand-alone ReLU kernel does, and packs y.  The pack's scale then comes from max|x|, an
// upper bound of max|y| that is known before the pass starts.
template <int TC, class E, bool RELU>
__global__ void __launch_bounds__(256) pack_nchw_kernel(const float* __restrict__ src, E* __restrict__ hi, E* __restrict__ lo, PackGeom g, ScaleRef sr,
                                                        float* __restrict__ y_out, AmaxOut am) {
  grid_dep_sync();
  // tile[c][f ^ (c / 8)]: the XOR keeps both phases free of bank conflicts (stores: 32 lanes = 32 frame positions
  // of one channel; loads: lanes = 8-channel groups of a few positions that are TC/8 apart)
  __shared__ float tile[TC][32];
  const float sc = pack_scale(sr, blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0);
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
  const int fsize = g.frame_h * g.frame_w;
  const int f0 = blockIdx.y * 32;                              // 32 consecutive frame positions (row-major over the frame)
  const int cblocks = (g.c_limit + TC - 1) / TC;               // blocks cover every column that has to be defined
  const int n = blockIdx.x / cblocks, c0 = (blockIdx.x % cblocks) * TC;
  {
    const int f = f0 + tx, i = f / g.frame_w, j = f - i * g.frame_w;
    const int si = i * g.sh - g.off_h, sj = j * g.sw - g.off_w;
    const bool ok = f < fsize && si >= 0 && si < g.H && sj >= 0 && sj < g.W;
    const long long plane = (long long)g.H * g.W;
    // one 64-bit address per thread, advanced by eight planes per load; the range checks are hoisted out of the
    // unrolled loads (a block whose channels all exist and a thread whose position has a source take the plain path)
    const float* sp = src + ((long long)n * g.C + c0 + ty) * plane + (long long)si * g.W + sj;
    const long long step = 8 * plane;
    const int avail = g.C - c0 - ty;                  // channels at or after this thread's first one
    float v[TC / 8];
    if (ok && c0 + TC <= g.C) {
#pragma unroll
      for (int k = 0; k < TC / 8; ++k) { v[k] = __ldg(sp); sp += step; }
    } else if (ok) {
#pragma unroll
      for (int k = 0; k < TC / 8; ++k) { v[k] = 8 * k < avail ? __ldg(sp) : 0.f; sp += step; }
    } else {
#pragma unroll
      for (int k = 0; k < TC / 8; ++k) v[k] = 0.f;
    }
    if (RELU) {
      uint32_t m = 0;
      if (ok) {
        float* yp = y_out + (sp - src) - (long long)(TC / 8) * step;        // the element the first load read
#pragma unroll
        for (int k = 0; k < TC / 8; ++k) {
          const float x = v[k];
          v[k] = x > 0.f ? x : (x != x ? x : 0.f);                           // NaN propagates
          if (8 * k < avail) { *yp = v[k]; m = max(m, amax_bits(v[k])); }
          yp += step;
        }
      }
      amax_commit(am, m);
    }
    float* trow = &tile[ty][0];
#pragma unroll
    for (int k = 0; k < TC / 8; ++k) trow[k * 8 * 32 + (tx ^ k)] = v[k] * sc;       // channel ty + 8k, column tx ^ ((ty + 8k) >> 3)
  }
  __syncthreads();
  {
    // a warp pass writes 32 / LPP whole pixels: lane -> (pixel slot, 8-channel group); 16-byte stores of hi and of lo
    constexpr int LPP = TC / 8;                       // lanes per pixel
    const int grp = tx % LPP, px = tx / LPP, cl = grp * 8, c = c0 + cl;
    for (int jb = ty; jb < LPP; jb += 8) {
      const int ff = jb + px * LPP, f = f0 + ff;
      if (f < fsize && c < g.c_limit) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = tile[cl + e][ff ^ grp];
        store8(hi, lo, ((long long)n * fsize + f) * g.pitch + g.dst_c0 + c, v);
      }
    }
  }
}

__device__ __forceinline__ void store_two(__half* p, __half a, __half b) { *reinterpret_cast<__half2*>(p) = __halves2half2(a, b); }
__device__ __forceinline__ void store_two(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
// NCHW activations -> explicit patch matrix [N*P*Q][pitch], column (c*R + r)*S + s = the filter's own flat index
// within one output channel, so the convolution becomes a 1x1 one over C*R*S "channels".  Used where the
// channel count is too small to fill a 64-wide reduction chunk per tap (first layers, C = 3).
struct PatchGeom { int N, C, H, W, R, S, P, Q, sh, sw, pad_h, pad_w, cols, pitch; };
template <class E>
__global__ void __launch_bounds__(256) pack_patches_kernel(const float* __restrict__ src, E* __restrict__ hi, E* __restrict__ lo, PatchGeom g, ScaleRef sr) {
  grid_dep_sync();
  // column -> (source offset relative to the window origin, r, s), the same for every row
  __shared__ int col_off[1024];
  __shared__ short col_r[1024], col_s[1024];
  const float sc = pack_scale(sr, blockIdx.x == 0 && threadIdx.x == 0);
  const int rs = g.R * g.S;
  for (int col = threadIdx.x; col < g.cols; col += blockDim.x) {
    const int c = col / rs, t = col - c * rs, r = t / g.S, q = t - r * g.S;
    col_off[col] = (c * g.H + r) * g.W + q;
    col_r[col] = (short)r; col_s[col] = (short)q;
  }
  __syncthreads();
  const long long rows = (long long)g.N * g.P * g.Q;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int pq = g.P * g.Q;
  for (long long row = (long long)blockIdx.x * wpb + warp; row < rows; row += (long long)gridDim.x * wpb) {   // one warp per patch row
    const int n = (int)(row / pq), rem = (int)(row - (long long)n * pq), pp = rem / g.Q, qq = rem - pp * g.Q;
    const int i0 = pp * g.sh - g.pad_h, j0 = qq * g.sw - g.pad_w;
    const float* base = src + ((long long)n * g.C * g.H + i0) * g.W + j0;
    const bool interior = i0 >= 0 && i0 + g.R <= g.H && j0 >= 0 && j0 + g.S <= g.W;
    E* h_row = hi + row * g.pitch;
    E* l_row = lo + row * g.pitch;
    for (int col2 = lane; col2 < g.pitch / 2; col2 += 32) {        // two columns per lane
      float a[2];
      if (interior) {          // the whole window lies inside the image (uniform over the warp): no per-tap range checks
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = 2 * col2 + e;
          a[e] = col < g.cols ? __ldg(base + col_off[col]) * sc : 0.f;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = 2 * col2 + e;
          a[e] = 0.f;
          if (col < g.cols) {
            const int i = i0 + col_r[col], j = j0 + col_s[col];
            if (i >= 0 && i < g.H && j >= 0 && j < g.W) a[e] = __ldg(base + col_off[col]) * sc;
          }
        }
      }
      E h0, l0, h1, l1;
      split_pair(a[0], h0, l0);
      split_pair(a[1], h1, l1);
      store_two(h_row + 2 * col2, h0, h1);
      store_two(l_row + 2 * col2, l0, l1);
    }
  }
}

// filters [K][C][R][S] -> forward pack [K][tap][cpad] (flip = 0) or backward-data pack [C][tap'][kpad] (flip = 1,
// tap' = (R-1-r)*S + (S-1-s)), zero in the channel padding.
template <class E>
__global__ void __launch_bounds__(256) pack_filter_kernel(const float* __restrict__ w, E* __restrict__ hi, E* __restrict__ lo,
                                                          int K, int C, int R, int S, int flip, int inner_pad, ScaleRef sr) {
  grid_dep_sync();
  const float sc = pack_scale(sr, blockIdx.x == 0 && threadIdx.x == 0);
  int taps = R * S;
  long long rows = flip ? C : K, total = rows * taps * inner_pad, stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    int in = (int)(idx % inner_pad);
    long long t2 = idx / inner_pad;
    int tap = (int)(t2 % taps), row = (int)(t2 / taps);
    int inner_n = flip ? K : C;
    float a = 0.f;
    if (in < inner_n) {
      int k = flip ? in : row, c = flip ? row : in;
      int src_tap = flip ? (taps - 1 - tap) : tap;
      a = w[((long long)k * C + c) * taps + src_tap] * sc;
    }
    E h, l;
    split_pair(a, h, l);
    hi[idx] = h; lo[idx] = l;
  }
}

// Both filter packs of one convolution in a single launch (the weights do not change between the forward and the
// backward-data call of a step, so the second pack rides along with the first): element idx of the forward pack and
// element idx of the backward-data pack per thread.
template <class E>
__global__ void __launch_bounds__(256) pack_filter_pair_kernel(const float* __restrict__ w, E* __restrict__ hi_f, E* __restrict__ lo_f,
                                                               E* __restrict__ hi_d, E* __restrict__ lo_d, int K, int C, int R, int S,
                                                               int pad_f, int pad_d, ScaleRef sr, float* __restrict__ scale_d) {
  grid_dep_sync();
  const bool first = blockIdx.x == 0 && threadIdx.x == 0;
  const float sc = pack_scale(sr, first);
  if (first) *scale_d = sc;
  const int taps = R * S;
  const long long total_f = (long long)K * taps * pad_f, total_d = (long long)C * taps * pad_d;
  const long long total = total_f > total_d ? total_f : total_d, stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    if (idx < total_f) {
      int in = (int)(idx % pad_f);
      long long t2 = idx / pad_f;
      int tap = (int)(t2 % taps), k = (int)(t2 / taps);
      float a = in < C ? w[((long long)k * C + in) * taps + tap] * sc : 0.f;
      E h, l;
      split_pair(a, h, l);
      hi_f[idx] = h; lo_f[idx] = l;
    }
    if (idx < total_d) {
      int in = (int)(idx % pad_d);
      long long t2 = idx / pad_d;
      int tap = (int)(t2 % taps), c = (int)(t2 / taps);
      float a = in < K ? w[((long long)in * C + c) * taps + (taps - 1 - tap)] * sc : 0.f;
      E h, l;
      split_pair(a, h, l);
      hi_d[idx] = h; lo_d[idx] = l;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}
static inline CUtensorMapDataType map_type(int ar) { return ar == kArithTF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16; }

// 2-D row-major [rows][cols] with `pitch` elements per row; box = one 128-byte row of K x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* m, int ar, const void* base, long long rows, long long cols, long long pitch, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  TF_REQUIRE(fn, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch * elem_of(ar)};
  cuuint32_t box[2] = {(cuuint32_t)bk_of(ar), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, map_type(ar), 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TF_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d (rows %lld cols %lld pitch %lld)", (int)r, rows, cols, pitch);
  return 0;
}
// M/N-major operand: 3-D view {group width, rows, pitch / group width column groups} (a group is 128 bytes of M/N) with
// a box of `tile_cols` columns x one stage of K rows.  The pack's pitch is a multiple of 64 elements, so every group lies
// inside the allocation; columns past the logical width only reach output rows / columns that the epilogue masks.
static int make_map_mn(CUtensorMap* m, int ar, const void* base, long long rows, long long pitch, int tile_cols) {
  EncodeTiledFn fn = encode_fn();
  TF_REQUIRE(fn, "cuTensorMapEncodeTiled is not available from this driver");
  const int gw = gw_of(ar);
  TF_REQUIRE(pitch % gw == 0 && tile_cols % gw == 0, "M/N-major operand: pitch %lld / tile width %d are not multiples of %d", pitch, tile_cols, gw);
  cuuint64_t dims[3] = {(cuuint64_t)gw, (cuuint64_t)rows, (cuuint64_t)(pitch / gw)};
  cuuint64_t strides[2] = {(cuuint64_t)pitch * elem_of(ar), 128};
  cuuint32_t box[3] = {(cuuint32_t)gw, (cuuint32_t)bk_of(ar), (cuuint32_t)(tile_cols / gw)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, map_type(ar), 3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  ar == kArithTF32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TF_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (3-D) failed with %d (rows %lld pitch %lld tile %d)", (int)r, rows, pitch, tile_cols);
  return 0;
}

// im2col-mode map over a halo-free pixel-major pack [N][H][W][pitch]: base pixels range over the box
// [-lo_w, W - lo_w' ) x [-lo_h, ...) that holds one base pixel per output position of a stride-1 window of
// win_w x win_h with lo_w / lo_h zero columns / rows in front (and as many behind as the output extent needs);
// a copy brings `pixels` base pixels x `chans` channels (128 bytes).
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
static EncodeIm2colFn encode_im2col_fn() {
  static EncodeIm2colFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return (EncodeIm2colFn)p;
  }();
  return fn;
}
static int make_map_im2col(CUtensorMap* m, int ar, const void* base, int N, int H, int W, long long pitch, int lo_w, int lo_h, int win_w, int win_h,
                           int pixels, int chans) {
  EncodeIm2colFn fn = encode_im2col_fn();
  TF_REQUIRE(fn, "cuTensorMapEncodeIm2col is not available from this driver");
  const int es = elem_of(ar);
  cuuint64_t dims[4] = {(cuuint64_t)pitch, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)pitch * es, (cuuint64_t)W * pitch * es, (cuuint64_t)H * W * pitch * es};
  int lower[2] = {-lo_w, -lo_h};
  int upper[2] = {lo_w - (win_w - 1), lo_h - (win_h - 1)};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, map_type(ar), 4, (void*)base, dims, strides, lower, upper, (cuuint32_t)chans, (cuuint32_t)pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TF_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeIm2col failed with %d (N %d H %d W %d pitch %lld lower %d,%d upper %d,%d)", (int)r, N, H, W, pitch, lower[0],
             lower[1], upper[0], upper[1]);
  return 0;
}

static std::mutex g_tc_mu;      // guards the lazily created process-wide state below
static int* error_word() {      // mapped pinned word: the kernels raise it, the host polls it for free
  static int* host = nullptr;
  static int* dev = nullptr;
  std::lock_guard<std::mutex> lk(g_tc_mu);
  if (!host) {
    if (cudaHostAlloc((void**)&host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) { cudaGetLastError(); host = nullptr; return nullptr; }
    *host = 0;
    if (cudaHostGetDevicePointer((void**)&dev, host, 0) != cudaSuccess) { cudaGetLastError(); dev = nullptr; }
  }
  return dev;
}
static int* error_word_host() {
  static std::atomic<int*> host{nullptr};
  int* h = host.load(std::memory_order_acquire);
  if (!h) {
    int* dev = error_word();
    if (!dev) return nullptr;
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, dev) == cudaSuccess) { h = (int*)at.hostPointer; host.store(h, std::memory_order_release); }
  }
  return h;
}
int tensor_path_error() { int* h = error_word_host(); return h ? *(volatile int*)h : 0; }
void tensor_path_error_clear() { int* h = error_word_host(); if (h) *(volatile int*)h = 0; }

int tensor_path_timeout_probe(long long limit_cycles, cudaStream_t s) {
  int* err = error_word();
  TF_REQUIRE(err, "the error word could not be mapped");
  TF_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000ll, "limit must be between 1 and 2e9 cycles");
  barrier_timeout_probe_kernel<<<1, 32, 0, s>>>(limit_cycles, err);
  return after_launch(s, "barrier_timeout_probe", 1);
}

// Arithmetic of the tensor path: 0 = 3xFP16 (scaled fp16 hi/lo pairs, kind::f16), 1 = 3xTF32 (tf32 hi/lo pairs, kind::tf32).
static std::atomic<int> g_arith{[] { const char* e = getenv("TINYFLOW_ARITH"); return (e && (!strcmp(e, "3xtf32") || !strcmp(e, "1"))) ? 1 : 0; }()};
int tensor_arithmetic() { return g_arith.load(std::memory_order_relaxed); }
void set_tensor_arithmetic(int a) { g_arith.store(a, std::memory_order_relaxed); }

// ---- schedule: whole waves of tiles, then the partial wave cut into equal per-CTA ranges of stages -------------------
// Costs are in units of one stage of one tile.  Splitting the tail pays a fixed price per CTA (the partial sums make a
// round trip through the workspace and a second kernel adds them), so it is taken only when the tail is clearly
// unbalanced and its reductions are long enough to share.
static float g_tail_gain = [] { const char* e = getenv("TINYFLOW_TAIL_GAIN"); return e ? (float)atof(e) : 0.9f; }();
static float g_tail_cost = [] { const char* e = getenv("TINYFLOW_TAIL_COST"); return e ? (float)atof(e) : 12.f; }();     // workspace round trip + second kernel, in stages
static int plan_schedule(GemmParams& g, int bn, cudaStream_t s, int* oom) {
  const int sms = device_sm_count();
  const int tiles = g.m_tiles * g.n_tiles * g.tap_tiles;
  g.full_tiles = tiles; g.tail_tiles = 0; g.tail_share = 0; g.slots_per_cta = 0; g.workspace = nullptr;
  const int rem = tiles % sms;
  static const bool no_split = getenv("TINYFLOW_NO_TAIL_SPLIT") != nullptr;
  if (rem == 0 || g.k_total < 8 || no_split) return 0;
  const long long units = (long long)rem * g.k_total;
  int share = (int)((units + sms - 1) / sms);
  if (share < 4) share = 4;                                   // shorter pieces are all overhead
  const double whole = g.k_total + 8.0, split = share + 8.0 + g_tail_cost;
  if (split >= g_tail_gain * whole) return 0;
  g.full_tiles = tiles - rem; g.tail_tiles = rem; g.tail_share = share;
  g.slots_per_cta = (share - 1 + g.k_total - 1) / g.k_total + 1;       // tiles a range of `share` stages can touch
  const int ctas = (int)((units + share - 1) / share);
  const size_t bytes = (size_t)ctas * g.slots_per_cta * bn * BM * sizeof(float);
  g.workspace = (float*)persistent_scratch(1, bytes);
  if (!g.workspace) { if (oom) *oom = bytes > 0x7fffffffu ? 0x7fffffff : (int)bytes; return 1; }
  (void)s;
  return 0;
}

static bool g_attr_done[2][3] = {{false, false, false}, {false, false, false}};
template <int BN, int AR> static int launch_gemm(const GemmParams& p, cudaStream_t s, double flops, const char* what) {
  using L = SmemLayout<BN>;
  constexpr int slot = BN == 64 ? 0 : (BN == 128 ? 1 : 2);
  {
    std::lock_guard<std::mutex> lk(g_tc_mu);
    if (!g_attr_done[AR][slot]) {
      TF_CUDA(cudaFuncSetAttribute(gemm3x_kernel<BN, AR>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      g_attr_done[AR][slot] = true;
    }
  }
  TF_REQUIRE(tensor_path_error() == 0, "%s: an earlier tensor-core kernel timed out on a barrier; refusing to launch", what);
  static const int group_iters = getenv("TINYFLOW_GROUP_ITERS") ? atoi(getenv("TINYFLOW_GROUP_ITERS")) : 0;
  const_cast<GemmParams&>(p).group_iters = group_iters > 0 ? group_iters : (p.data_by_data ? kGroupItersDataByData : (AR == kArithTF32 ? kGroupItersTF32 : kGroupIters));
  static const int acc_layout = getenv("TINYFLOW_ACC_LAYOUT") ? atoi(getenv("TINYFLOW_ACC_LAYOUT")) : 2;
  const_cast<GemmParams&>(p).acc_layout = acc_layout;
  const int sms = device_sm_count();
  const int tiles = p.full_tiles + p.tail_tiles;
  int grid = tiles < sms ? tiles : sms;
  if (p.tail_share > 0) {
    const int ctas = (int)(((long long)p.tail_tiles * p.k_total + p.tail_share - 1) / p.tail_share);
    grid = p.full_tiles > 0 ? sms : ctas;
  }
  note_compute_stream(s);
  static const bool detail = getenv("TINYFLOW_TIMING_DETAIL") != nullptr;    // one timing row per distinct problem shape
  char name[192];
  if (detail) snprintf(name, sizeof(name), "gemm3x%s mode%d M%d N%d ktotal%d taps%d bn%d tiles%d tail%d share%d %s", AR == kArithTF32 ? "tf32" : "f16", p.mode, p.M,
                       p.N, p.k_total, p.tap_tiles, BN, tiles, p.tail_tiles, p.tail_share, what + 5);
  KernelTimer kt(detail ? name : (AR == kArithTF32 ? "gemm3xtf32_tcgen05" : "gemm3xf16_tcgen05"), s, flops, 0, 1);
  launch_dep(gemm3x_kernel<BN, AR>, dim3(grid), dim3(kThreads), (size_t)L::kTotal, s, p);
  TF_AFTER(s, what);
  if (p.tail_share > 0) {
    launch_dep(reduce_partials_kernel<BN>, dim3(p.tail_tiles, BN / kReduceCols), dim3(BM, kReduceWays), 0, s, p);
    TF_AFTER(s, what);
  }
  return 0;
}
// CTA-pair launch: 74 clusters of two CTAs, programmatic dependent launch as everywhere else.
static bool g_pair_attr_done[2] = {false, false};
template <int AR> static int launch_gemm_pair(const GemmParams& p, cudaStream_t s, double flops, const char* what) {
  using L = PairLayout;
  {
    std::lock_guard<std::mutex> lk(g_tc_mu);
    if (!g_pair_attr_done[AR]) {
      TF_CUDA(cudaFuncSetAttribute(gemm3x_pair_kernel<AR>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      g_pair_attr_done[AR] = true;
    }
  }
  TF_REQUIRE(tensor_path_error() == 0, "%s: an earlier tensor-core kernel timed out on a barrier; refusing to launch", what);
  static const int group_iters = getenv("TINYFLOW_GROUP_ITERS") ? atoi(getenv("TINYFLOW_GROUP_ITERS")) : 0;
  const_cast<GemmParams&>(p).group_iters = group_iters > 0 ? group_iters : (p.data_by_data ? kGroupItersDataByData : (AR == kArithTF32 ? kGroupItersTF32 : kGroupIters));
  const int pair_tiles = ((p.m_tiles + 1) / 2) * p.n_tiles * p.tap_tiles;
  const int pairs = std::min(device_sm_count() / 2, pair_tiles);
  note_compute_stream(s);
  static const bool detail = getenv("TINYFLOW_TIMING_DETAIL") != nullptr;
  static const bool no_dep = getenv("TINYFLOW_NO_DEPENDENT_LAUNCH") != nullptr;
  char name[192];
  if (detail) snprintf(name, sizeof(name), "gemm3x%s pairs mode%d M%d N%d ktotal%d pairtiles%d %s", AR == kArithTF32 ? "tf32" : "f16", p.mode, p.M, p.N, p.k_total, pair_tiles, what + 5);
  KernelTimer kt(detail ? name : (AR == kArithTF32 ? "gemm3xtf32_tcgen05" : "gemm3xf16_tcgen05"), s, flops, 0, 1);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = (size_t)L::kTotal; cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  memset(attrs, 0, sizeof(attrs));
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs; cfg.numAttrs = (no_dep || s == (cudaStream_t)0) ? 1 : 2;
  TF_CUDA(cudaLaunchKernelEx(&cfg, gemm3x_pair_kernel<AR>, p));
  TF_AFTER(s, what);
  return 0;
}
// Pairs pay where the one-CTA kernel waits for operands: K-major operands, 128-column tiles, reductions of at least 8
// stages, and enough 256-row tiles to occupy the 74 pairs.
static int g_pairs_mode = [] { const char* e = getenv("TINYFLOW_PAIRS"); return e ? atoi(e) : 0; }();
static bool pairs_wanted(int bn, int m_tiles, int n_tiles, int k_total) {
  if (g_pairs_mode == 0 || bn != 128) return false;
  if (g_pairs_mode >= 2) return true;                   // 2: wherever the kernel can run (tests)
  return k_total >= 8 && ((m_tiles + 1) / 2) * n_tiles >= 60;
}
template <int AR> static int launch_gemm_ar(int bn, const GemmParams& p, cudaStream_t s, double flops, const char* what) {
  return bn == 64 ? launch_gemm<64, AR>(p, s, flops, what) : bn == 96 ? launch_gemm<96, AR>(p, s, flops, what) : launch_gemm<128, AR>(p, s, flops, what);
}
// Plans the schedule (which may need workspace) and launches.  Returns 0 on success, -1 on error, 1 when the workspace
// could not be allocated (*oom holds the byte count).
static int launch_gemm_bn(int bn, int ar, GemmParams& p, cudaStream_t s, double flops, const char* what, int* oom) {
  if (int rc = plan_schedule(p, bn, s, oom)) return rc;
  return ar == kArithTF32 ? launch_gemm_ar<kArithTF32>(bn, p, s, flops, what) : launch_gemm_ar<kArithF16>(bn, p, s, flops, what);
}
// N-tile width.  M/N-major B operands come in 64-column groups, so they take 64 or 128; K-major ones may also take
// 96, which wastes less on widths such as 96, 160, 192 or 288.
static inline int pick_bn(long long n, bool b_k_major = false) {
  if (n <= 64) return 64;
  if (!b_k_major) return 128;
  long long w128 = (n + 127) / 128 * 128, w96 = (n + 95) / 96 * 96;
  return w96 < w128 ? 96 : 128;
}
static inline long long round_up(long long a, long long b) { return (a + b - 1) / b * b; }

struct Pack {           // a packed operand living in pooled device memory
  void* hi = nullptr; void* lo = nullptr;
  uint32_t* words = nullptr;       // device: amax[0], amax[1] (alternating between uses), scale (float), spare
  unsigned uses = 0;
  int arith = kArithF16;           // element type of hi / lo
  long long rows = 0, cols = 0, pitch = 0;
  const void* src = nullptr; uint64_t version = 0; int tag = 0;   // cache key
  size_t bytes() const { return (size_t)rows * pitch * elem_of(arith); }
  const float* scale() const { return reinterpret_cast<const float*>(words + 2); }
};
static int pack_alloc(Pack& pk, int ar, long long rows, long long cols, cudaStream_t s, int* oom) {
  long long pitch = round_up(cols, 64);
  if (!pk.words) {
    pk.words = (uint32_t*)pool_alloc(16);
    if (!pk.words || cudaMemsetAsync(pk.words, 0, 16, s) != cudaSuccess) { if (oom) *oom = 16; return 1; }
    pk.uses = 0;
  }
  if (pk.hi && pk.rows == rows && pk.pitch == pitch && pk.arith == ar) { pk.cols = cols; return 0; }
  if (pk.hi) { pool_free(pk.hi); pool_free(pk.lo); pk.hi = pk.lo = nullptr; }
  pk.rows = rows; pk.cols = cols; pk.pitch = pitch; pk.src = nullptr; pk.arith = ar;
  pk.hi = pool_alloc(pk.bytes());
  pk.lo = pk.hi ? pool_alloc(pk.bytes()) : nullptr;
  if (!pk.lo) {
    if (pk.hi) pool_free(pk.hi);
    pk.hi = nullptr;
    if (oom) *oom = pk.bytes() > 0x7fffffffu ? 0x7fffffff : (int)pk.bytes();
    return 1;
  }
  return 0;
}
static void pack_release(Pack& pk) {
  if (pk.hi) { pool_free(pk.hi); pool_free(pk.lo); pk.hi = pk.lo = nullptr; }
  if (pk.words) { pool_free(pk.words); pk.words = nullptr; }
}
// Starts one use of the pack: reduces max|src| over n contiguous floats into this use's amax word and returns the
// references the pack kernel needs.  Several pack launches of the same use (stride phases) share one ScaleRef.
// A tf32 pack needs no maximum: its scale is 1.
static ScaleRef begin_pack(Pack& pk, const float* src, long long n, cudaStream_t s) {
  if (pk.arith == kArithTF32) return ScaleRef{nullptr, nullptr, reinterpret_cast<float*>(pk.words + 2)};
  const unsigned k = pk.uses++ & 1;
  ScaleRef r{pk.words + k, pk.words + (k ^ 1), reinterpret_cast<float*>(pk.words + 2)};
  static const bool no_track = getenv("TINYFLOW_NO_AMAX_TRACKING") != nullptr;
  if (const uint32_t* tracked = no_track ? nullptr : amax_tracked(src)) {
    r.amax_cur = tracked;               // the producer of src already reduced max|src| in its own pass
    return r;
  }
  KernelTimer kt("amax", s, 0, 4.0 * n);
  launch_dep(amax_kernel, dim3(grid_for(n, 256, 32)), dim3(256), 0, s, src, n, pk.words + k);
  return r;
}
// Calls `fn(hi, lo)` with the pack's buffers typed by its element type.
template <class F> static void with_elems(const Pack& pk, F&& fn) {
  if (pk.arith == kArithTF32) fn((float*)pk.hi, (float*)pk.lo);
  else fn((__half*)pk.hi, (__half*)pk.lo);
}

static int run_pack_matrix(const float* src, long long ld, Pack& pk, cudaStream_t s) {
  long long total = pk.rows * pk.cols;
  ScaleRef sr = begin_pack(pk, src, total, s);          // callers pass ld == cols: the matrix is contiguous
  KernelTimer kt("pack_matrix", s, 0, 4.0 * total + 2.0 * elem_of(pk.arith) * total);
  const bool vec = pk.cols % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  with_elems(pk, [&](auto* hi, auto* lo) {
    using E = std::remove_pointer_t<decltype(hi)>;
    if (vec) launch_dep(pack_matrix_kernel<true, E>, dim3(grid_for(total / 8, 256, 2)), dim3(256), 0, s, src, ld, hi, lo, pk.pitch, pk.rows, pk.cols, sr);
    else launch_dep(pack_matrix_kernel<false, E>, dim3(grid_for(total, 256, 4)), dim3(256), 0, s, src, ld, hi, lo, pk.pitch, pk.rows, pk.cols, sr);
  });
  TF_AFTER(s, "pack_matrix");
  return 0;
}

// ---- matmul ---------------------------------------------------------------------------------------
int tc_matmul(const float* A, bool tA, const float* B, bool tB, float* C, int64_t M, int64_t N, int64_t K, cudaStream_t s, int* oom) {
  if (M < 16 || N < 16 || K < 64 || (double)M * N * K < 4e6) return 0;      // launch-bound sizes stay on the CUDA cores
  if (!encode_fn()) return 0;
  const int ar = tensor_arithmetic(), bk = bk_of(ar);
  // A is stored [M][K] (K-major) or, transposed, [K][M] (M-major); B is stored [K][N] (N-major) or [N][K] (K-major)
  Pack pa, pb;
  long long a_rows = tA ? K : M, a_cols = tA ? M : K, b_rows = tB ? N : K, b_cols = tB ? K : N;
  if (pack_alloc(pa, ar, a_rows, a_cols, s, oom)) { pack_release(pa); return 0; }
  if (pack_alloc(pb, ar, b_rows, b_cols, s, oom)) { pack_release(pa); pack_release(pb); return 0; }
  int rc = run_pack_matrix(A, a_cols, pa, s);
  if (!rc) rc = run_pack_matrix(B, b_cols, pb, s);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int bn = pick_bn(N, tB);
  p.mode = kModeGemm; p.a_mn = tA ? 1 : 0; p.b_mn = tB ? 0 : 1; p.epi = kEpiRowMajor;
  p.data_by_data = tA ? 1 : 0;     // A^T B is how a dense layer's weight gradient (X^T dY) arrives
  if (!rc) rc = p.a_mn ? make_map_mn(&p.a_hi, ar, pa.hi, pa.rows, pa.pitch, BM) : make_map(&p.a_hi, ar, pa.hi, pa.rows, pa.cols, pa.pitch, BM);
  if (!rc) rc = p.a_mn ? make_map_mn(&p.a_lo, ar, pa.lo, pa.rows, pa.pitch, BM) : make_map(&p.a_lo, ar, pa.lo, pa.rows, pa.cols, pa.pitch, BM);
  if (!rc) rc = p.b_mn ? make_map_mn(&p.b_hi, ar, pb.hi, pb.rows, pb.pitch, bn) : make_map(&p.b_hi, ar, pb.hi, pb.rows, pb.cols, pb.pitch, bn);
  if (!rc) rc = p.b_mn ? make_map_mn(&p.b_lo, ar, pb.lo, pb.rows, pb.pitch, bn) : make_map(&p.b_lo, ar, pb.lo, pb.rows, pb.cols, pb.pitch, bn);
  if (!rc) {
    p.M = (int)M; p.N = (int)N;
    p.m_tiles = (int)((M + BM - 1) / BM); p.n_tiles = (int)((N + bn - 1) / bn); p.tap_tiles = 1;
    p.k_total = (int)((K + bk - 1) / bk);
    p.out = C; p.ldc = N; p.err = error_word();
    p.a_scale = pa.scale(); p.b_scale = pb.scale();
    rc = launch_gemm_bn(bn, ar, p, s, 2.0 * M * N * K, "DLGpuMatrixMultiply", oom);
  }
  pack_release(pa); pack_release(pb);       // stream order keeps the blocks valid until the kernel is done
  return rc < 0 ? -1 : (rc > 0 ? 0 : 1);    // a missing workspace sends the call to the CUDA-core kernel
}

// ---- convolution -------------------------------------------------------------------------------------
// Shapes the tensor path takes (everything else returns 0 and runs on the CUDA cores):
//   class A: 1x1 window, no padding, any stride (frame = the P x Q output grid, x sampled with the stride);
//   class B: stride 1, padding <= window - 1 on each axis, any window: frame = (H + R - 1) x (W + S - 1); x sits at
//            offset (pad_h, pad_w), dy at (R - 1 - pad_h, S - 1 - pad_w), which gives each the zero halo its role
//            needs (forward padding for x, "full" correlation for dy);
//   class D: strided windows: space-to-depth phases (see conv_state);
//   class C: too few input channels for a per-tap reduction chunk: x is expanded into patches (C*R*S columns) and
//            the problem runs as class A over C*R*S channels; forward and filter gradient only.
struct ConvTc {
  int cls = 0;                 // 0 unsupported, 1 class A, 2 class B, 3 class C, 4 class D
  int frame_h = 0, frame_w = 0;                          // frame geometry shared by the x and dy packs
  int x_off_h = 0, x_off_w = 0, dy_off_h = 0, dy_off_w = 0;
  int eC = 0, eR = 1, eS = 1;                            // reduction channels and window of the problem as the GEMM sees it
  int cp = 0;                                            // class D: columns per stride phase (C rounded up to 64)
  bool dgrad_seen = false;                               // backward-data has run on this plan: forward also packs its filter layout
  Pack x, dy, wf, wd;
  std::mutex mu;
};
static ConvTc* conv_state(ConvPlan* p) {
  if (!p->tc_state) {
    ConvTc* st = new ConvTc;
    st->eC = p->C; st->eR = p->R; st->eS = p->S;
    bool base = p->dataformat == 0 && p->K >= 16 && p->K % 4 == 0 && p->R * p->S <= kMaxTaps;
    bool ok = base && p->C >= 16 && p->C % 4 == 0;
    if (ok && p->R == 1 && p->S == 1 && p->pad_h == 0 && p->pad_w == 0) {
      st->cls = 1; st->frame_h = p->P; st->frame_w = p->Q;
    } else if (ok && p->stride_h == 1 && p->stride_w == 1 && p->pad_h <= p->R - 1 && p->pad_w <= p->S - 1) {
      st->cls = 2;
      static const bool shared_halo = [] { const char* e = getenv("TINYFLOW_SHARED_HALO"); return e ? atoi(e) != 0 : true; }();
      if (shared_halo) {
        // x and dy both sit at the frame's origin and the frame is only max(pad, window-1-pad) wider / taller than the
        // input: a tap that reaches left of column 0 lands in the zero gap that ends the previous frame row (right of
        // the last column: the gap of its own row), above row 0 in the zero rows that end the previous image (or before
        // the pack: zero fill).  The gap is shared by both sides, so the frame has (H+g)(W+g) positions instead of
        // (H+R-1)(W+S-1): 1.31x the outputs instead of 1.65x at 7x7 with a 3x3 window.
        const int gh = std::max(p->pad_h, p->R - 1 - p->pad_h), gw = std::max(p->pad_w, p->S - 1 - p->pad_w);
        st->frame_h = p->H + gh; st->frame_w = p->W + gw;
      } else {
        st->frame_h = p->H + p->R - 1; st->frame_w = p->W + p->S - 1;
        st->x_off_h = p->pad_h; st->x_off_w = p->pad_w; st->dy_off_h = p->R - 1 - p->pad_h; st->dy_off_w = p->S - 1 - p->pad_w;
      }
    } else if (ok && p->stride_h * p->stride_w <= 16 && p->pad_h <= p->R - 1 && p->pad_w <= p->S - 1 &&
               (long long)p->stride_h * p->stride_w * round_up(p->C, 64) < 32768) {
      // strided window: x is split into stride_h*stride_w phases (space to depth), each tap reads one phase at a
      // stride-1 shift; dy sits behind a halo of (R-1)/stride_h, (S-1)/stride_w for the backward-data pass
      st->cls = 4; st->cp = (int)round_up(p->C, 64);
      st->dy_off_h = (p->R - 1) / p->stride_h; st->dy_off_w = (p->S - 1) / p->stride_w;
      int uh = (p->H - 1 + p->pad_h) / p->stride_h + 1, uw = (p->W - 1 + p->pad_w) / p->stride_w + 1;
      st->frame_h = (uh > p->P ? uh : p->P) + st->dy_off_h; st->frame_w = (uw > p->Q ? uw : p->Q) + st->dy_off_w;
    } else if (base && p->C < 16 && p->C * p->R * p->S <= 1024) {
      st->cls = 3; st->frame_h = p->P; st->frame_w = p->Q;
      st->eC = p->C * p->R * p->S; st->eR = st->eS = 1;
    }
    // small problems are launch-bound: leave them to the CUDA-core kernel
    double flops = 2.0 * p->N * p->K * p->P * p->Q * p->C * p->R * p->S;
    if (flops < 2e7) st->cls = 0;
    p->tc_state = st;
  }
  return (ConvTc*)p->tc_state;
}

// One launch of the frame pack: `chans` channels of an NCHW tensor (spatial dims H x W) into columns dst_c0 .. dst_c0 + cover
// of pk (zeros past `chans`)
static int launch_pack_nchw(Pack& pk, const ScaleRef& sr, const float* src, int N, int chans, int H, int W, int frame_h, int frame_w, int off_h, int off_w,
                            int sh, int sw, int dst_c0, int cover, cudaStream_t s, float* relu_out = nullptr, AmaxOut relu_am = AmaxOut{}) {
  PackGeom g{N, chans, H, W, frame_h, frame_w, off_h, off_w, sh, sw, (int)pk.pitch, dst_c0, cover};
  const int tc = cover > 64 ? 128 : cover > 32 ? 64 : 32;
  dim3 grid(N * ((cover + tc - 1) / tc), (frame_h * frame_w + 31) / 32);
  TF_REQUIRE(grid.y <= 65535, "pack: frame of %d x %d positions is too large", frame_h, frame_w);
  KernelTimer kt(relu_out ? "relu_pack" : "pack_nchw", s, 0, (relu_out ? 8.0 : 4.0) * N * chans * H * W / (sh * sw) + 2.0 * elem_of(pk.arith) * pk.rows * cover);
  with_elems(pk, [&](auto* hi, auto* lo) {
    using E = std::remove_pointer_t<decltype(hi)>;
    if (relu_out) {
      if (tc == 128) launch_dep(pack_nchw_kernel<128, E, true>, grid, dim3(256), 0, s, src, hi, lo, g, sr, relu_out, relu_am);
      else if (tc == 64) launch_dep(pack_nchw_kernel<64, E, true>, grid, dim3(256), 0, s, src, hi, lo, g, sr, relu_out, relu_am);
      else launch_dep(pack_nchw_kernel<32, E, true>, grid, dim3(256), 0, s, src, hi, lo, g, sr, relu_out, relu_am);
    } else {
      if (tc == 128) launch_dep(pack_nchw_kernel<128, E, false>, grid, dim3(256), 0, s, src, hi, lo, g, sr, (float*)nullptr, AmaxOut{});
      else if (tc == 64) launch_dep(pack_nchw_kernel<64, E, false>, grid, dim3(256), 0, s, src, hi, lo, g, sr, (float*)nullptr, AmaxOut{});
      else launch_dep(pack_nchw_kernel<32, E, false>, grid, dim3(256), 0, s, src, hi, lo, g, sr, (float*)nullptr, AmaxOut{});
    }
  });
  TF_AFTER(s, relu_out ? "relu_pack" : "pack_nchw");
  return 0;
}
static bool pack_valid(const Pack& pk, int ar, const void* src, uint64_t ver, int tag, long long rows, long long cols) {
  return pk.hi && pk.arith == ar && pk.src == src && pk.version == ver && pk.tag == tag && pk.rows == rows && pk.cols == cols;
}
// ---- producers that write a consumer's pack ---------------------------------------------------------------------------
// The graph calls BN -> ReLU -> convolution as separate entry points, and the convolution then re-reads the ReLU's output
// to pack it.  Every ReLU call that comes with a descriptor (one per graph node, stable from step to step) leaves a note
// "this address was written by that node"; when a frame pack of x is made, the node that wrote x is looked up and the
// plan is remembered under the node.  From the next step on that node's ReLU packs its output for the plan in the same
// pass (relu_pack), whatever address the executor hands it, and the convolution finds the pack valid.  A wrong guess
// costs one unused pack.
struct PackTarget { ConvTc* st; int N, C, H, W; };
static std::atomic<long long> g_fused_relu_packs{0};
static std::mutex g_targets_mu;
struct ReluNote { const void* node; uint64_t version; };
static std::unordered_map<const void*, ReluNote> g_relu_writer;             // output address -> the ReLU node that wrote it, and the write version it left
static std::unordered_map<const void*, PackTarget> g_pack_targets;          // ReLU descriptor -> plan that packs its output
void tc_note_relu_output(const void* node, const void* y) {     // call after the output's write version was bumped
  if (!node) return;
  const uint64_t ver = version_of(y);
  std::lock_guard<std::mutex> lk(g_targets_mu);
  g_relu_writer[y] = ReluNote{node, ver};
}
static void remember_pack_target(const void* x, uint64_t ver, ConvTc* st, const ConvPlan* p) {
  std::lock_guard<std::mutex> lk(g_targets_mu);
  auto it = g_relu_writer.find(x);
  if (it != g_relu_writer.end() && it->second.version == ver) g_pack_targets[it->second.node] = PackTarget{st, p->N, p->C, p->H, p->W};
}

// the x operand of a plan: frame pack (classes A, B), patch matrix (class C) or one frame per stride phase (class D)
static int pack_x(ConvTc* st, int ar, const ConvPlan* p, const float* x, cudaStream_t s, int* oom) {
  Pack& pk = st->x;
  const uint64_t ver = version_of(x);
  const long long n_src = (long long)p->N * p->C * p->H * p->W;
  if (st->cls == 3) {
    long long rows = (long long)p->N * p->P * p->Q;
    if (pack_valid(pk, ar, x, ver, 3, rows, st->eC)) return 0;
    if (pack_alloc(pk, ar, rows, st->eC, s, oom)) return 1;
    ScaleRef sr = begin_pack(pk, x, n_src, s);
    PatchGeom g{p->N, p->C, p->H, p->W, p->R, p->S, p->P, p->Q, p->stride_h, p->stride_w, p->pad_h, p->pad_w, st->eC, (int)pk.pitch};
    KernelTimer kt("pack_patches", s, 0, 2.0 * elem_of(ar) * rows * pk.pitch);
    with_elems(pk, [&](auto* hi, auto* lo) {
      using E = std::remove_pointer_t<decltype(hi)>;
      launch_dep(pack_patches_kernel<E>, dim3(grid_for(rows * 32, 256, 4)), dim3(256), 0, s, x, hi, lo, g, sr);
    });
    TF_AFTER(s, "pack_patches");
    pk.src = x; pk.version = ver; pk.tag = 3;
    return 0;
  }
  const long long rows = (long long)p->N * st->frame_h * st->frame_w;
  const int phases = st->cls == 4 ? p->stride_h * p->stride_w : 1;
  const long long cols = st->cls == 4 ? (long long)phases * st->cp : p->C;
  if (pack_valid(pk, ar, x, ver, st->cls, rows, cols)) return 0;
  if (pack_alloc(pk, ar, rows, cols, s, oom)) return 1;
  ScaleRef sr = begin_pack(pk, x, n_src, s);
  int rc = 0;
  if (st->cls == 4) {
    // phase (a, b) holds x_padded(sh*u + a, sw*v + b) = x(sh*u + a - pad_h, sw*v + b - pad_w) at frame position (u, v)
    for (int a = 0; a < p->stride_h && !rc; ++a)
      for (int b = 0; b < p->stride_w && !rc; ++b) {
        int ph = a * p->stride_w + b;
        rc = launch_pack_nchw(pk, sr, x, p->N, p->C, p->H, p->W, st->frame_h, st->frame_w, p->pad_h - a, p->pad_w - b, p->stride_h, p->stride_w, ph * st->cp, st->cp, s);
      }
  } else {
    rc = launch_pack_nchw(pk, sr, x, p->N, p->C, p->H, p->W, st->frame_h, st->frame_w, st->x_off_h, st->x_off_w, p->stride_h, p->stride_w, 0, (int)pk.pitch, s);
  }
  if (rc) return -1;
  pk.src = x; pk.version = ver; pk.tag = st->cls;
  if ((st->cls == 1 || st->cls == 2) && p->stride_h == 1 && p->stride_w == 1) remember_pack_target(x, ver, st, p);
  return 0;
}
static int pack_dy(ConvTc* st, int ar, const ConvPlan* p, const float* dy, cudaStream_t s, int* oom) {
  Pack& pk = st->dy;
  const uint64_t ver = version_of(dy);
  const long long rows = (long long)p->N * st->frame_h * st->frame_w;
  if (pack_valid(pk, ar, dy, ver, 2, rows, p->K)) return 0;
  if (pack_alloc(pk, ar, rows, p->K, s, oom)) return 1;
  ScaleRef sr = begin_pack(pk, dy, (long long)p->N * p->K * p->P * p->Q, s);
  if (launch_pack_nchw(pk, sr, dy, p->N, p->K, p->P, p->Q, st->frame_h, st->frame_w, st->dy_off_h, st->dy_off_w, 1, 1, 0, (int)pk.pitch, s)) return -1;
  pk.src = dy; pk.version = ver; pk.tag = 2;
  return 0;
}
// Halo-free pixel-major packs [N][H][W][C] of x and [N][P][Q][K] of dy for the im2col route (tags 20 / 21)
static int pack_plain(Pack& pk, int ar, int tag, const float* src, int N, int chans, int H, int W, cudaStream_t s, int* oom) {
  const uint64_t ver = version_of(src);
  const long long rows = (long long)N * H * W;
  if (pack_valid(pk, ar, src, ver, tag, rows, chans)) return 0;
  if (pack_alloc(pk, ar, rows, chans, s, oom)) return 1;
  ScaleRef sr = begin_pack(pk, src, rows * chans, s);
  if (launch_pack_nchw(pk, sr, src, N, chans, H, W, H, W, 0, 0, 1, 1, 0, (int)pk.pitch, s)) return -1;
  pk.src = src; pk.version = ver; pk.tag = tag;
  return 0;
}
// Filter packs are keyed like the activation packs (pointer, write version): an optimiser step bumps the version.
// `with_other` makes the forward call produce the backward-data pack in the same launch.
static int pack_filter(ConvTc* st, int ar, const float* w, const ConvPlan* p, int flip, bool with_other, cudaStream_t s, int* oom) {
  Pack& pk = flip ? st->wd : st->wf;
  const uint64_t ver = version_of(w);
  const int taps = st->eR * st->eS;
  auto dims = [&](int f, int& rows, int& pad) { rows = f ? st->eC : p->K; pad = (int)round_up(f ? p->K : st->eC, 64); };
  int rows, pad;
  dims(flip, rows, pad);
  if (pack_valid(pk, ar, w, ver, 10 + flip, rows, (long long)taps * pad)) return 0;
  if (pack_alloc(pk, ar, rows, (long long)taps * pad, s, oom)) return 1;
  const long long nw = (long long)p->K * p->C * p->R * p->S;
  if (with_other && !flip) {
    Pack& pd = st->wd;
    int rows_d, pad_d;
    dims(1, rows_d, pad_d);
    if (pack_alloc(pd, ar, rows_d, (long long)taps * pad_d, s, oom)) return 1;
    ScaleRef sr = begin_pack(pk, w, nw, s);
    long long total = std::max((long long)rows * taps * pad, (long long)rows_d * taps * pad_d);
    with_elems(pk, [&](auto* hi, auto* lo) {
      using E = std::remove_pointer_t<decltype(hi)>;
      launch_dep(pack_filter_pair_kernel<E>, dim3(grid_for(total, 256)), dim3(256), 0, s, w, hi, lo, (E*)pd.hi, (E*)pd.lo, p->K, st->eC, st->eR, st->eS, pad, pad_d, sr,
                 reinterpret_cast<float*>(pd.words + 2));
    });
    TF_AFTER(s, "pack_filter");
    pk.src = w; pk.version = ver; pk.tag = 10;
    pd.src = w; pd.version = ver; pd.tag = 11;
    return 0;
  }
  ScaleRef sr = begin_pack(pk, w, nw, s);
  long long total = (long long)rows * taps * pad;
  with_elems(pk, [&](auto* hi, auto* lo) {
    using E = std::remove_pointer_t<decltype(hi)>;
    launch_dep(pack_filter_kernel<E>, dim3(grid_for(total, 256)), dim3(256), 0, s, w, hi, lo, p->K, st->eC, st->eR, st->eS, flip, pad, sr);
  });
  TF_AFTER(s, "pack_filter");
  pk.src = w; pk.version = ver; pk.tag = 10 + flip;
  return 0;
}

// forward and backward-data share one launcher: out[pixel][ch_out] = sum_{tap, ch_in} act[pixel + off(tap)][col(tap) + ch_in] * filt[ch_out][b(tap)][ch_in]
struct TapList { int n = 0; int off[kMaxTaps]; int col[kMaxTaps]; int b[kMaxTaps]; void add(int o, int c, int bb) { off[n] = o; col[n] = c; b[n] = bb; ++n; } };
struct OutGeom { int valid_h, valid_w, out_h, out_w, out_sh, out_sw, out_off_h, out_off_w; };
// returns 0 on success, -1 on error, 1 when scratch memory was short (*oom set)
// Geometry of an im2col read of the activation pack: the pack is [N][H][W][pitch]; a stride-1 window of win_w x win_h
// with lo_w / lo_h zero columns / rows in front gives box_w x box_h base pixels (= output positions) per image.
struct Im2colGeom { int N, H, W, lo_w, lo_h, win_w, win_h, box_w, box_h; };
static int conv_like(const Pack& act, const Pack& filt, int ch_in, int ch_out, int frame_h, int frame_w, float* out, const TapList& taps,
                     const OutGeom& og, double flops, cudaStream_t s, const char* what, int* oom, const Im2colGeom* im = nullptr) {
  GemmParams g;
  memset(&g, 0, sizeof(g));
  const int ar = act.arith, bk = bk_of(ar);
  const int bn = pick_bn(ch_out, true);
  g.mode = kModeConv; g.epi = kEpiNchw;
  int rc;
  if (im) {
    rc = make_map_im2col(&g.a_hi, ar, act.hi, im->N, im->H, im->W, act.pitch, im->lo_w, im->lo_h, im->win_w, im->win_h, BM, bk);
    if (!rc) rc = make_map_im2col(&g.a_lo, ar, act.lo, im->N, im->H, im->W, act.pitch, im->lo_w, im->lo_h, im->win_w, im->win_h, BM, bk);
    g.im2col = 1; g.im_w = im->box_w; g.im_h = im->box_h; g.im_lo_w = -im->lo_w; g.im_lo_h = -im->lo_h;
  } else {
    rc = make_map(&g.a_hi, ar, act.hi, act.rows, act.cols, act.pitch, BM);
    if (!rc) rc = make_map(&g.a_lo, ar, act.lo, act.rows, act.cols, act.pitch, BM);
  }
  const long long m_rows = im ? (long long)im->N * im->box_w * im->box_h : act.rows;      // one GEMM row per output position
  const bool pairs = !im && pairs_wanted(bn, (int)((m_rows + BM - 1) / BM), (ch_out + bn - 1) / bn, taps.n * ((ch_in + bk - 1) / bk));
  if (!rc) rc = make_map(&g.b_hi, ar, filt.hi, filt.rows, filt.cols, filt.pitch, pairs ? bn / 2 : bn);      // a pair's CTAs load half a B tile each
  if (!rc) rc = make_map(&g.b_lo, ar, filt.lo, filt.rows, filt.cols, filt.pitch, pairs ? bn / 2 : bn);
  if (rc) return -1;
  g.M = (int)m_rows; g.N = ch_out;
  g.m_tiles = (int)((m_rows + BM - 1) / BM); g.n_tiles = (ch_out + bn - 1) / bn; g.tap_tiles = 1;
  g.ntaps = taps.n;
  g.chunks_per_tap = (ch_in + bk - 1) / bk;
  g.b_tap_pitch = (int)round_up(ch_in, 64);
  g.k_total = g.ntaps * g.chunks_per_tap;
  for (int t = 0; t < taps.n; ++t) { g.tap_off[t] = taps.off[t]; g.tap_col[t] = (short)taps.col[t]; g.tap_b[t] = (short)taps.b[t]; }
  g.out = out; g.err = error_word();
  g.a_scale = act.scale(); g.b_scale = filt.scale();
  g.frame_h = frame_h; g.frame_w = frame_w; g.valid_h = og.valid_h; g.valid_w = og.valid_w;
  g.out_c = ch_out; g.out_h = og.out_h; g.out_w = og.out_w; g.out_sh = og.out_sh; g.out_sw = og.out_sw; g.out_off_h = og.out_off_h; g.out_off_w = og.out_off_w;
  if (pairs) return ar == kArithTF32 ? launch_gemm_pair<kArithTF32>(g, s, flops, what) : launch_gemm_pair<kArithF16>(g, s, flops, what);
  return launch_gemm_bn(bn, ar, g, s, flops, what, oom);
}
static double conv_flops(const ConvPlan* p) { return 2.0 * p->N * p->K * p->P * p->Q * p->C * p->R * p->S; }
// Stride-1 windows (class B) in the fp16 arithmetic read halo-free packs through im2col tensor maps: the GEMM's rows are
// the real output positions only (a halo frame spends (H+R-1)(W+S-1)/(HW) times the multiplies, 1.65x at 7x7), and the
// packs are smaller.  TINYFLOW_IM2COL=0 keeps the halo frames.
static bool use_im2col(const ConvTc* st, int ar) {
  static const bool on = [] { const char* e = getenv("TINYFLOW_IM2COL"); return e ? atoi(e) != 0 : false; }();
  return on && st->cls == 2 && ar == kArithF16 && encode_im2col_fn() != nullptr;
}
// window offsets of every tap, packed as (r << 16) | s
static void im2col_taps(TapList& taps, int R, int S) {
  for (int r = 0; r < R; ++r) for (int q = 0; q < S; ++q) taps.add((r << 16) | q, 0, r * S + q);
}
// result of a tensor-path entry point from the launcher's code
static inline int tc_result(int rc) { return rc < 0 ? -1 : (rc > 0 ? 1 : 1); }

// ReLU forward (graph node `node`: the address of its descriptor) whose output the tensor path is expected to pack next:
// y = relu(x) and the consumer plan's frame pack of y in one pass.  Returns 1 when it did that, 0 when the caller should run the plain ReLU (no known consumer, or in the
// fp16 arithmetic no recorded max|x| to bound the scale with), -1 on error.
int tc_fused_relu_pack(const void* node, const float* x, float* y, int64_t n, cudaStream_t s) {
  static const bool on = [] { const char* e = getenv("TINYFLOW_FUSE_RELU_PACK"); return e ? atoi(e) != 0 : true; }();
  if (!on || !node || contraction_path_is_cuda_cores()) return 0;
  PackTarget t;
  {
    std::lock_guard<std::mutex> lk(g_targets_mu);
    auto it = g_pack_targets.find(node);
    if (it == g_pack_targets.end()) return 0;
    t = it->second;
  }
  if ((int64_t)t.N * t.C * t.H * t.W != n || x == y) return 0;
  const int ar = tensor_arithmetic();
  ConvTc* st = t.st;
  if (use_im2col(st, ar)) return 0;
  const uint32_t* bound = ar == kArithF16 ? amax_tracked(x) : nullptr;
  if (ar == kArithF16 && !bound) return 0;
  std::lock_guard<std::mutex> lk(st->mu);
  Pack& pk = st->x;
  int oom = 0;
  const long long rows = (long long)t.N * st->frame_h * st->frame_w;
  if (pack_alloc(pk, ar, rows, t.C, s, &oom)) return 0;
  note_write(y);
  AmaxOut am = amax_track_begin(y);
  ScaleRef sr{bound, nullptr, reinterpret_cast<float*>(pk.words + 2)};       // scale from max|x| >= max|relu(x)|; tf32: no scale
  note_compute_stream(s);
  if (launch_pack_nchw(pk, sr, x, t.N, t.C, t.H, t.W, st->frame_h, st->frame_w, st->x_off_h, st->x_off_w, 1, 1, 0, (int)pk.pitch, s, y, am)) return -1;
  pk.src = y; pk.version = version_of(y); pk.tag = st->cls;
  tc_note_relu_output(node, y);
  g_fused_relu_packs.fetch_add(1, std::memory_order_relaxed);
  return 1;
}
long long fused_relu_pack_count() { return g_fused_relu_packs.load(std::memory_order_relaxed); }

int tc_conv_fwd(ConvPlan* p, const float* x, const float* w, float* y, cudaStream_t s, int* oom) {
  ConvTc* st = conv_state(p);
  if (!st->cls || !encode_fn()) return 0;
  const int ar = tensor_arithmetic();
  std::lock_guard<std::mutex> lk(st->mu);
  if (use_im2col(st, ar)) {
    if (pack_plain(st->x, ar, 20, x, p->N, p->C, p->H, p->W, s, oom)) return *oom ? 1 : -1;
    if (pack_filter(st, ar, w, p, 0, st->dgrad_seen, s, oom)) return *oom ? 1 : -1;
    TapList taps;
    im2col_taps(taps, p->R, p->S);
    Im2colGeom im{p->N, p->H, p->W, p->pad_w, p->pad_h, p->S, p->R, p->Q, p->P};
    OutGeom og{p->P, p->Q, p->P, p->Q, 1, 1, 0, 0};
    return tc_result(conv_like(st->x, st->wf, st->eC, p->K, p->P, p->Q, y, taps, og, conv_flops(p), s, "DLGpuConvolution2DForward", oom, &im));
  }
  if (pack_x(st, ar, p, x, s, oom)) return *oom ? 1 : -1;
  if (pack_filter(st, ar, w, p, 0, st->dgrad_seen, s, oom)) return *oom ? 1 : -1;
  TapList taps;
  for (int r = 0; r < st->eR; ++r)
    for (int q = 0; q < st->eS; ++q) {
      if (st->cls == 4) taps.add((r / p->stride_h) * st->frame_w + q / p->stride_w, ((r % p->stride_h) * p->stride_w + q % p->stride_w) * st->cp, r * st->eS + q);
      else if (st->cls == 2) taps.add((r - p->pad_h + st->x_off_h) * st->frame_w + (q - p->pad_w + st->x_off_w), 0, r * st->eS + q);   // output (p, q) is anchored at frame position (p, q)
      else taps.add(r * st->frame_w + q, 0, r * st->eS + q);
    }
  OutGeom og{p->P, p->Q, p->P, p->Q, 1, 1, 0, 0};
  return tc_result(conv_like(st->x, st->wf, st->eC, p->K, st->frame_h, st->frame_w, y, taps, og, conv_flops(p), s, "DLGpuConvolution2DForward", oom));
}

int tc_conv_dgrad(ConvPlan* p, const float* dy, const float* w, float* dx, cudaStream_t s, int* oom) {
  ConvTc* st = conv_state(p);
  if (!st->cls || st->cls == 3 || !encode_fn()) return 0;
  const int ar = tensor_arithmetic();
  std::lock_guard<std::mutex> lk(st->mu);
  if (use_im2col(st, ar)) {
    // dx = correlation of dy with the flipped filter, R-1-pad zero rows / columns in front
    if (pack_plain(st->dy, ar, 21, dy, p->N, p->K, p->P, p->Q, s, oom)) return *oom ? 1 : -1;
    st->dgrad_seen = true;
    if (pack_filter(st, ar, w, p, 1, false, s, oom)) return *oom ? 1 : -1;
    TapList taps;
    im2col_taps(taps, p->R, p->S);
    Im2colGeom im{p->N, p->P, p->Q, p->S - 1 - p->pad_w, p->R - 1 - p->pad_h, p->S, p->R, p->W, p->H};
    OutGeom og{p->H, p->W, p->H, p->W, 1, 1, 0, 0};
    return tc_result(conv_like(st->dy, st->wd, p->K, p->C, p->H, p->W, dx, taps, og, conv_flops(p), s, "DLGpuConvolutionBackwardData", oom, &im));
  }
  if (pack_dy(st, ar, p, dy, s, oom)) return *oom ? 1 : -1;
  st->dgrad_seen = true;                                           // from now on forward packs both layouts in one launch
  if (pack_filter(st, ar, w, p, 1, false, s, oom)) return *oom ? 1 : -1;     // [C][flipped tap][K]; a no-op when forward made it
  const int ntap = p->R * p->S;
  int rc = 0;
  if (st->cls == 1) {
    // a strided 1x1 window reaches only every stride-th input position: the rest of dx is zero
    bool strided = p->stride_h > 1 || p->stride_w > 1;
    if (strided && cudaMemsetAsync(dx, 0, sizeof(float) * (size_t)p->N * p->C * p->H * p->W, s) != cudaSuccess) return -1;
    TapList taps; taps.add(0, 0, 0);
    OutGeom og{p->P, p->Q, p->H, p->W, p->stride_h, p->stride_w, 0, 0};
    rc = conv_like(st->dy, st->wd, p->K, p->C, st->frame_h, st->frame_w, dx, taps, og, conv_flops(p), s, "DLGpuConvolutionBackwardData", oom);
  } else if (st->cls == 2) {
    TapList taps;
    // dx(h, w), anchored at frame position (h, w), reads dy(h - lo_h + r, w - lo_w + s) with lo = window - 1 - pad
    for (int r = 0; r < p->R; ++r)
      for (int q = 0; q < p->S; ++q)
        taps.add((r - (p->R - 1 - p->pad_h) + st->dy_off_h) * st->frame_w + (q - (p->S - 1 - p->pad_w) + st->dy_off_w), 0, r * p->S + q);
    OutGeom og{p->H, p->W, p->H, p->W, 1, 1, 0, 0};
    rc = conv_like(st->dy, st->wd, p->K, p->C, st->frame_h, st->frame_w, dx, taps, og, conv_flops(p), s, "DLGpuConvolutionBackwardData", oom);
  } else {
    // One launch per stride phase (a, b): dx_padded(sh*u + a, sw*v + b) = sum over the taps r = sh*r' + a, s = sw*s' + b of
    // dy(u - r', v - s') * w(r, s); dy sits at frame offset (hh, hw), so the shift is (hh - r') rows and (hw - s') columns.
    // The phases write disjoint positions of dx; positions no phase reaches stay zero.
    if (cudaMemsetAsync(dx, 0, sizeof(float) * (size_t)p->N * p->C * p->H * p->W, s) != cudaSuccess) return -1;
    for (int a = 0; a < p->stride_h && !rc; ++a)
      for (int b = 0; b < p->stride_w && !rc; ++b) {
        TapList taps;
        for (int r = a; r < p->R; r += p->stride_h)
          for (int q = b; q < p->S; q += p->stride_w)
            taps.add((st->dy_off_h - r / p->stride_h) * st->frame_w + (st->dy_off_w - q / p->stride_w), 0, ntap - 1 - (r * p->S + q));
        if (!taps.n) continue;      // no tap lands on this phase: it stays zero
        OutGeom og{st->frame_h, st->frame_w, p->H, p->W, p->stride_h, p->stride_w, a - p->pad_h, b - p->pad_w};
        rc = conv_like(st->dy, st->wd, p->K, p->C, st->frame_h, st->frame_w, dx, taps, og, conv_flops(p) * taps.n / ntap, s, "DLGpuConvolutionBackwardData", oom);
      }
  }
  return tc_result(rc);
}

int tc_conv_wgrad(ConvPlan* p, const float* x, const float* dy, float* dw, cudaStream_t s, int* oom) {
  ConvTc* st = conv_state(p);
  if (!st->cls || !encode_fn()) return 0;
  const int ar = tensor_arithmetic(), bk = bk_of(ar);
  std::lock_guard<std::mutex> lk(st->mu);
  if (use_im2col(st, ar)) {
    // dW[k][c][r][s] = sum over output pixels of dy[pixel][k] * x[pixel + (r, s) - pad][c]: the reduction runs over the
    // real output pixels; x comes through an im2col map (BK pixels x one 128-byte channel group per copy), dy as it lies
    if (pack_plain(st->x, ar, 20, x, p->N, p->C, p->H, p->W, s, oom)) return *oom ? 1 : -1;
    if (pack_plain(st->dy, ar, 21, dy, p->N, p->K, p->P, p->Q, s, oom)) return *oom ? 1 : -1;
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.err = error_word(); g.out = dw; g.data_by_data = 1;
    const int bn = pick_bn(p->K);
    g.mode = kModeWgrad; g.a_mn = 1; g.b_mn = 1; g.epi = kEpiWgrad;
    g.M = p->C; g.N = p->K; g.ntaps = p->R * p->S;
    g.slot = p->C > 64 ? BM : 64;
    g.taps_per_tile = BM / g.slot;
    int rc = make_map_im2col(&g.a_hi, ar, st->x.hi, p->N, p->H, p->W, st->x.pitch, p->pad_w, p->pad_h, p->S, p->R, bk, gw_of(ar));
    if (!rc) rc = make_map_im2col(&g.a_lo, ar, st->x.lo, p->N, p->H, p->W, st->x.pitch, p->pad_w, p->pad_h, p->S, p->R, bk, gw_of(ar));
    if (!rc) rc = make_map_mn(&g.b_hi, ar, st->dy.hi, st->dy.rows, st->dy.pitch, bn);
    if (!rc) rc = make_map_mn(&g.b_lo, ar, st->dy.lo, st->dy.rows, st->dy.pitch, bn);
    if (rc) return -1;
    g.a_scale = st->x.scale(); g.b_scale = st->dy.scale();
    g.m_tiles = (p->C + g.slot - 1) / g.slot;
    g.tap_tiles = (g.ntaps + g.taps_per_tile - 1) / g.taps_per_tile;
    g.n_tiles = (p->K + bn - 1) / bn;
    g.im2col = 1; g.im_w = p->Q; g.im_h = p->P; g.im_lo_w = -p->pad_w; g.im_lo_h = -p->pad_h;
    for (int r = 0; r < p->R; ++r) for (int q = 0; q < p->S; ++q) g.tap_off[r * p->S + q] = (r << 16) | q;
    g.k_total = (int)((st->dy.rows + bk - 1) / bk);
    return tc_result(launch_gemm_bn(bn, ar, g, s, conv_flops(p), "DLGpuConvolutionBackwardFilter", oom));
  }
  if (pack_x(st, ar, p, x, s, oom)) return *oom ? 1 : -1;
  if (pack_dy(st, ar, p, dy, s, oom)) return *oom ? 1 : -1;
  GemmParams g;
  memset(&g, 0, sizeof(g));
  g.err = error_word(); g.out = dw; g.data_by_data = 1;
  const int kit = (int)((st->dy.rows + bk - 1) / bk);       // the reduction runs over the frame's pixel rows
  if (st->eR * st->eS == 1 && st->dy_off_h == 0 && st->dy_off_w == 0) {
    // One tap: dW[k][c] = dy^T x is a plain GEMM over the two packs, and either operand may take the M side.
    // Take the orientation whose padded tile grid is smaller (64 input channels would fill half of a 128-row tile).
    auto padded = [](long long m, long long n) { int b = pick_bn(n); return ((m + BM - 1) / BM * BM) * ((n + b - 1) / b * b); };
    const long long slot_rows = st->eC > 64 ? (st->eC + BM - 1) / BM * BM : BM;
    const int bn_x = pick_bn(p->K);
    const long long as_is = slot_rows * ((p->K + bn_x - 1) / bn_x * bn_x);
    if (padded(p->K, st->eC) < as_is) {
      const int bn = pick_bn(st->eC);
      g.mode = kModeGemm; g.a_mn = 1; g.b_mn = 1; g.epi = kEpiRowMajor;
      int rc = make_map_mn(&g.a_hi, ar, st->dy.hi, st->dy.rows, st->dy.pitch, BM);
      if (!rc) rc = make_map_mn(&g.a_lo, ar, st->dy.lo, st->dy.rows, st->dy.pitch, BM);
      if (!rc) rc = make_map_mn(&g.b_hi, ar, st->x.hi, st->x.rows, st->x.pitch, bn);
      if (!rc) rc = make_map_mn(&g.b_lo, ar, st->x.lo, st->x.rows, st->x.pitch, bn);
      if (rc) return -1;
      g.a_scale = st->dy.scale(); g.b_scale = st->x.scale();
      g.M = p->K; g.N = st->eC; g.ldc = st->eC;
      g.m_tiles = (p->K + BM - 1) / BM; g.n_tiles = (st->eC + bn - 1) / bn; g.tap_tiles = 1; g.ntaps = 1;
      g.k_total = kit;
      return tc_result(launch_gemm_bn(bn, ar, g, s, conv_flops(p), "DLGpuConvolutionBackwardFilter", oom));
    }
  }
  // A = x (M = tap slots x input channels), B = dy (N = output channels); both M/N-major, reduction over pixel rows.
  const int bn = pick_bn(p->K);
  g.mode = kModeWgrad; g.a_mn = 1; g.b_mn = 1; g.epi = kEpiWgrad;
  g.M = st->eC; g.N = p->K; g.ntaps = st->eR * st->eS;
  // Few input channels: two filter taps share one 128-row tile (slots of 64 channels), so that the tensor core's
  // M dimension is full and dy is read once for both.
  g.slot = st->eC > 64 ? BM : 64;
  g.taps_per_tile = BM / g.slot;
  int rc = make_map_mn(&g.a_hi, ar, st->x.hi, st->x.rows, st->x.pitch, g.slot);
  if (!rc) rc = make_map_mn(&g.a_lo, ar, st->x.lo, st->x.rows, st->x.pitch, g.slot);
  if (!rc) rc = make_map_mn(&g.b_hi, ar, st->dy.hi, st->dy.rows, st->dy.pitch, bn);
  if (!rc) rc = make_map_mn(&g.b_lo, ar, st->dy.lo, st->dy.rows, st->dy.pitch, bn);
  if (rc) return -1;
  g.a_scale = st->x.scale(); g.b_scale = st->dy.scale();
  g.m_tiles = (st->eC + g.slot - 1) / g.slot;
  g.tap_tiles = (g.ntaps + g.taps_per_tile - 1) / g.taps_per_tile;
  g.n_tiles = (p->K + bn - 1) / bn;
  // dy row m' holds output pixel (p, q) at frame position (p + dy_off_h, q + dy_off_w); tap (r, s) needs the padded
  // input at (p + r, q + s), which sits at frame row m' + (r - dy_off_h) * frame_w + (s - dy_off_w)
  for (int r = 0; r < st->eR; ++r)
    for (int q = 0; q < st->eS; ++q) {
      int t = r * st->eS + q;
      if (st->cls == 4) {
        g.tap_off[t] = (r / p->stride_h - st->dy_off_h) * st->frame_w + (q / p->stride_w - st->dy_off_w);
        g.tap_col[t] = (short)(((r % p->stride_h) * p->stride_w + q % p->stride_w) * st->cp);
      } else {
        const int ph = st->cls == 2 ? p->pad_h : st->x_off_h, pw = st->cls == 2 ? p->pad_w : st->x_off_w;    // classes A / C: no padding, offsets 0
        g.tap_off[t] = (r - ph + st->x_off_h - st->dy_off_h) * st->frame_w + (q - pw + st->x_off_w - st->dy_off_w);
      }
    }
  g.k_total = kit;
  return tc_result(launch_gemm_bn(bn, ar, g, s, conv_flops(p), "DLGpuConvolutionBackwardFilter", oom));
}

}  // namespace tf
