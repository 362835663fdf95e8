// Host-callable launchers of the sm_100a kernels.  This header is plain C++
// (no ATen, no CUDA headers beyond the runtime API types) so that the backend
// sources compile with the host compiler and the .cu files compile without
// pulling in torch.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace mccl {
namespace kern {

constexpr int kMaxWorld = 8;         // ranks sharing one NVSwitch domain
constexpr int kMaxCtas = 128;        // upper bound on CTAs of one collective kernel (signal-pad rows)
constexpr int kMaxCtasPerLane = 64;  // what a launcher may use: two lanes x 64 CTAs stay co-resident on 148 SMs
constexpr int kNumPhases = 4;        // independent signal arrays per lane
constexpr int kNumLanes = 2;         // collectives of consecutive epochs may run concurrently (one per lane)
constexpr int kNumParity = 4;        // data buffers per arena: epoch e uses buffer e % 4

enum DType : int { F32 = 0, F64, F16, BF16, I32, I64, U8, BOOL, DTYPE_COUNT };
enum RedOp : int { SUM = 0, AVG, MIN, MAX, PRODUCT, REDOP_COUNT };

inline size_t dtype_size(DType t) {
  switch (t) {
    case F32: case I32: return 4;
    case F64: case I64: return 8;
    case F16: case BF16: return 2;
    default: return 1;
  }
}

// ---- symmetric arena layout -------------------------------------------------
// Every rank owns one arena:  [ signal pad | data buffer 0 | ... | data buffer 3 ].
// Epoch e runs in lane e % 2 (lanes map to two communication streams, so two
// consecutive collectives overlap) and uses data buffer e % 4.
// The signal pad holds 32-bit epoch flags, all written remotely with release
// semantics and polled locally with acquire semantics:
//   entered[lane][src]        src has started epoch `seq` of that lane (buffer-reuse credit)
//   sig[lane][phase][cta][src] src's CTA `cta` finished phase `phase` of `seq`
// Flags only ever grow (the epoch is the process group's arena sequence
// number), so they are never reset and a late reader can not miss a value.
constexpr size_t kSignalBytes = 64 * 1024;
constexpr size_t kEnteredOffset = 0;                         // u32[kNumLanes][kMaxWorld]
constexpr size_t kSigOffset = 256;                           // u32[kNumLanes][kNumPhases][kMaxCtas][kMaxWorld]
static_assert(kSigOffset + size_t(kNumLanes) * kNumPhases * kMaxCtas * kMaxWorld * 4 <= kSignalBytes,
              "signal pad too small");

// Device status block (device memory, one per process group; the host reads it
// with an asynchronous copy on a side stream).
// word 0: 0 = healthy, else an ErrorCode; 1: seq; 2: phase; 3: peer waited for.
enum ErrorCode : uint32_t { ERR_NONE = 0, ERR_WAIT_TIMEOUT = 1, ERR_BOUNDS = 2 };
constexpr int kStatusWords = 8;
constexpr int kStatusMirrorWord = 4;  // words 4-5: device address of a host-mapped copy of words 0-3 (0: none)
// Phase stamps (ns, %globaltimer) of the last collective, written by CTA 0:
// 0 kernel start, 1 entered, 2 push done, 3 peers' pushes seen, 4 reduce done,
// 5 peers' reduces seen, 6 pull done / end.
constexpr int kStampSlots = 8;
constexpr int kMaxTilesPerCta = 1024;  // pipelined kernels publish a 12-bit running tile count

struct RankCtx {
  int rank;
  int ws;
  char* arena[kMaxWorld];  // arena base of every rank as mapped here; arena[rank] is local
  const void* in;          // this rank's input  (user tensor)
  void* out;               // this rank's output (user tensor)
  uint32_t* status;        // kStatusWords words
  unsigned long long* stamps;  // optional: kStampSlots globaltimer stamps written by CTA 0 (nullptr = off)
  // NVLS region (nullptr when the group has none): the same physical buffers of every rank, seen
  // through this rank's own mapping (nvls_uc: plain loads/stores hit local memory only) and through
  // the NVSwitch multicast mapping (nvls_mc: multimem.st reaches every rank's copy,
  // multimem.ld_reduce returns the sum over all ranks' copies).
  char* nvls_uc;
  char* nvls_mc;
};

struct CollParams {
  RankCtx ctx[kMaxWorld];  // real launch: ctx[0] only (grid.y == 1); emulation: one per rank
  uint32_t seq;            // arena epoch of this collective (same on every rank)
  size_t parity_offset;    // byte offset of this epoch's data buffer inside the arena
  size_t parity_capacity;  // bytes available in it
  int64_t count;           // elements (meaning depends on the collective)
  int root;                // broadcast root
  int op;                  // RedOp
  float scale;             // multiplied into the result (1/world for AVG, DDP pre-division...)
  unsigned long long wait_ns;  // bound on every in-kernel wait
  int tiles;               // two-shot: pipeline tiles per CTA (<=1: bulk phases)
  int64_t chunk_pitch;     // reduce_scatter: elements between the starts of consecutive input chunks (0: count)
  int push_gather;         // two-shot allreduce: owners push reduced chunks (needs 2x arena) instead of peers pulling
  int64_t out_pitch;       // allgather: bytes between the starts of consecutive ranks' blocks in `out` (0: count)
  int tile_bytes;          // pipelined byte movers / NVLS kernels: bytes per pipeline tile (0: built-in default)
  size_t nvls_offset;      // byte offset of this epoch's buffer inside the NVLS region
  size_t nvls_capacity;    // bytes available in it
  int use_nvls;            // byte movers: move the payload with multimem.st through the NVLS region
  int debug_checks;        // verify every computed offset against the buffer bounds; a violation is
                           // reported as ERR_BOUNDS in the status block and the access is skipped
};

struct LaunchCfg {
  int ctas = 0;     // 0: pick from the message size
  int threads = 512;
  int emulate_ranks = 0;  // >0: single-device emulation, grid.y = ranks, cooperative launch
};

// Picks the CTA count for `bytes` of payload (identical on every rank).
int pick_ctas(size_t bytes, int ws, int requested);

// Arena-size requirements (bytes of one parity buffer) for a payload.
size_t oneshot_arena_bytes(size_t nbytes, int ws);
size_t twoshot_arena_bytes(size_t nbytes, int ws, bool push_gather = false);
size_t allgather_stage_bytes(size_t nbytes_per_rank, int ws);  // staging space of one allgather launch
size_t broadcast_stage_bytes(size_t nbytes);
size_t nvls_allreduce_stage_bytes(size_t nbytes_wire, int ws);
// Tile geometry the pipelined kernels derive for (units, grid); exposed for host-side checks.
void tile_plan_host(int64_t units, int nctas, int nthreads, int64_t tile_bytes, int64_t* tile_units, int64_t* ntiles);
// The tile size the byte movers (allgather, two-hop broadcast) use for `units` 16-byte units of one
// rank's block on `nctas` CTAs at world size `ws` (test hook for the rule in coll_common.cuh).
int64_t mover_tile_bytes_host(int64_t units, int nctas, int64_t tile_bytes, int ws);

// All launchers return cudaSuccess or the launch error; none synchronises.
// dtype: element type of in/out.  wire: element type stored in the arena
// (== dtype, or F16/BF16 when dtype is F32: fused wire cast).
cudaError_t launch_allreduce_oneshot(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                     cudaStream_t s);
cudaError_t launch_allreduce_twoshot(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                     cudaStream_t s);
// ctx.in = ws concatenated chunks of `count` elements, ctx.out = `count` elements.
cudaError_t launch_reduce_scatter(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                  cudaStream_t s);
// Byte movers: count = bytes per rank.  allgather: out holds ws * count bytes.
cudaError_t launch_allgather(const CollParams& p, LaunchCfg cfg, cudaStream_t s);
cudaError_t launch_broadcast(const CollParams& p, LaunchCfg cfg, cudaStream_t s);
cudaError_t launch_barrier(const CollParams& p, LaunchCfg cfg, cudaStream_t s);
// SUM / AVG allreduce through the NVLS region (multimem.ld_reduce + multimem.st).  Supported
// (dtype, wire): F32/F32, F16/F16, BF16/BF16, F32/BF16, F32/F16; anything else returns
// cudaErrorNotSupported before launching.
bool nvls_allreduce_supported(DType dtype, DType wire, int op);
// In place on a tensor that lives in multicast-bound memory: ctx[0].nvls_uc / nvls_mc are the bases of
// that memory, nvls_offset the tensor's offset in it; count * sizeof(dtype) must be a multiple of 16.
cudaError_t launch_allreduce_nvls_inplace(const CollParams& p, DType dtype, LaunchCfg cfg, cudaStream_t s);
// `split`: the two local staging passes run as separate full-grid kernels around the kernel
// that talks to the peers (large messages); otherwise one tile-pipelined kernel does all three.
cudaError_t launch_allreduce_nvls(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg, cudaStream_t s,
                                  bool split = false);

// ---- standalone elementwise kernels (test hooks + local paths) ---------------
cudaError_t launch_ew_reduce(void* dst, const void* src, int64_t n, DType t, RedOp op, cudaStream_t s);
cudaError_t launch_ew_scale(void* buf, int64_t n, DType t, double scale, cudaStream_t s);
cudaError_t launch_ew_accumulate_scale(void* dst, const void* src, int64_t n, DType t, double scale,
                                       cudaStream_t s);
// dst(wire dtype) = cast(src(fp32)) and back.
cudaError_t launch_cast(void* dst, DType dt, const void* src, DType st, int64_t n, float scale,
                        cudaStream_t s);

}  // namespace kern
}  // namespace mccl
