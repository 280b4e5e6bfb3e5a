// Sum of the gradient bucket over the replicas of a data-parallel job, through peer memory
// (NVLink / NVSwitch), as one kernel per GPU that can be recorded in the CUDA graph of a step.
// It is the device form of what the data-parallel driver otherwise does with one NCCL all-reduce
// between two graphs: edge::merge_grads over all replicas (tiny_dnn/network.h:880-906 sums the
// per-sample gradients of ONE mini-batch; replicas extend that sum across GPUs, with no 1/N).
//
// Every rank owns a buffer that all ranks have mapped ("symmetric" memory):
//   slots[2][world][npad] floats, then flags[2][PR_CHUNKS] counters
// A step uses the half `step & 1`.  Block b of every rank
//   1. pushes chunk b of its own bucket into slot [rank] of EVERY rank's buffer (plain peer stores),
//   2. makes the stores visible (system fence) and adds 1 to flag b of every rank,
//   3. waits until its own flag b has received `world` additions for this use of the half,
//   4. sums the `world` slots of chunk b in rank order -- the same order on every rank, so the
//      replicas stay bit-identical -- into the local bucket.
// No block waits for another block of its own GPU, every wait is bounded by wall time (a timeout
// sets the context's error word and leaves the bucket untouched), and the half is reused only two
// steps later, after every rank has passed the step in between.  Every load is CTA-local or a plain
// load of this GPU's own memory; the peers are only written.
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

namespace {

constexpr int PR_CHUNKS = 128;   // blocks: all resident at once on 148 SMs
constexpr int PR_THREADS = 256;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerArgs {
  float *grads;              // local bucket, n floats: read, then overwritten with the sum
  float *const *bases;       // [world] base of every rank's buffer as mapped here
  const unsigned *step;      // number of reductions done so far
  int *err;
  int rank, world;
  long long n, npad, chunk;  // floats; npad and chunk are multiples of 4
};

__global__ void __launch_bounds__(PR_THREADS) peer_reduce_kernel(const PeerArgs a) {
  __shared__ int s_fail;
  const int tid = threadIdx.x, b = blockIdx.x;
  const unsigned step = *a.step;
  const int half = (int)(step & 1u);
  const unsigned target = (step / 2u + 1u) * (unsigned)a.world;  // additions this flag has seen after this use
  const long long c0 = (long long)b * a.chunk;
  const long long c1 = c0 + a.chunk < a.n ? c0 + a.chunk : a.n;
  const size_t flag_off = (size_t)2 * a.world * a.npad;          // floats before the flags
  const size_t my_slot = ((size_t)half * a.world + a.rank) * a.npad;
  // 1. push this rank's chunk into every rank's buffer
  for (long long i = c0 + 4 * tid; i < c1; i += 4 * PR_THREADS) {
    if (i + 4 <= c1) {
      const float4 v = *reinterpret_cast<const float4 *>(a.grads + i);
      for (int p = 0; p < a.world; ++p) *reinterpret_cast<float4 *>(a.bases[p] + my_slot + i) = v;
    } else {
      for (long long j = i; j < c1; ++j) {
        const float v = a.grads[j];
        for (int p = 0; p < a.world; ++p) a.bases[p][my_slot + j] = v;
      }
    }
  }
  // 2. publish, then signal every rank
  __threadfence_system();
  __syncthreads();
  if (tid < a.world) {
    unsigned *flag = reinterpret_cast<unsigned *>(a.bases[tid] + flag_off) + half * PR_CHUNKS + b;
    __threadfence_system();  // the signalling thread itself orders the block's stores (seen through the barrier) before the flag
    atomicAdd_system(flag, 1u);
  }
  // 3. wait for every rank's chunk (bounded: about two seconds of wall time)
  if (tid == 0) {
    const unsigned *mine = reinterpret_cast<const unsigned *>(a.bases[a.rank] + flag_off) + half * PR_CHUNKS + b;
    int fail = 0;
    if (ld_acquire_sys(mine) < target) {
      unsigned long long t0, t1;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
      for (;;) {
        bool done = false;
        for (int k = 0; k < 64 && !done; ++k) done = ld_acquire_sys(mine) >= target;
        if (done) break;
        asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) {
          fail = 1;
          break;
        }
      }
    }
    s_fail = fail;
  }
  __syncthreads();
  if (s_fail) {
    if (tid == 0 && a.err) atomicExch(a.err, 7);
    return;
  }
  // 4. sum the slots in rank order; the peers' stores sit in this GPU's memory / L2, not in this SM's L1
  const float *slots = a.bases[a.rank] + (size_t)half * a.world * a.npad;
  for (long long i = c0 + 4 * tid; i < c1; i += 4 * PR_THREADS) {
    if (i + 4 <= c1) {
      float4 s = __ldcg(reinterpret_cast<const float4 *>(slots + i));
      for (int r = 1; r < a.world; ++r) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(slots + (size_t)r * a.npad + i));
        s.x = __fadd_rn(s.x, v.x);
        s.y = __fadd_rn(s.y, v.y);
        s.z = __fadd_rn(s.z, v.z);
        s.w = __fadd_rn(s.w, v.w);
      }
      *reinterpret_cast<float4 *>(a.grads + i) = s;
    } else {
      for (long long j = i; j < c1; ++j) {
        float s = __ldcg(slots + j);
        for (int r = 1; r < a.world; ++r) s = __fadd_rn(s, __ldcg(slots + (size_t)r * a.npad + j));
        a.grads[j] = s;
      }
    }
  }
}

__global__ void peer_advance_kernel(unsigned *step) { *step += 1u; }

long long pr_npad(long long n) { return (n + 3) / 4 * 4; }

}  // namespace

// bytes of the buffer every rank must provide (zero-filled, mapped by all ranks)
size_t peer_reduce_bytes(long long n, int world) {
  return ((size_t)2 * world * pr_npad(n)) * sizeof(float) + (size_t)2 * PR_CHUNKS * sizeof(unsigned);
}

int peer_reduce_init(b200_ctx *ctx, PeerReduce *pr, long long n, int rank, int world,
                     const unsigned long long *bases) {
  B200_REQUIRE(world >= 2 && world <= PR_THREADS && rank >= 0 && rank < world && n > 0 && bases,
               "peer_reduce_init: bad argument");
  for (int p = 0; p < world; ++p)
    B200_REQUIRE(bases[p] != 0 && (bases[p] & 15) == 0, "peer_reduce_init: buffer of rank %d is NULL or unaligned", p);
  peer_reduce_free(pr);
  pr->rank = rank;
  pr->world = world;
  pr->n = n;
  B200_CUDA(cudaMalloc(&pr->bases_dev, sizeof(float *) * world));
  B200_CUDA(cudaMemcpy(pr->bases_dev, bases, sizeof(float *) * world, cudaMemcpyHostToDevice));
  B200_CUDA(cudaMalloc(&pr->step_dev, sizeof(unsigned)));
  B200_CUDA(cudaMemset(pr->step_dev, 0, sizeof(unsigned)));
  (void)ctx;
  return 0;
}

void peer_reduce_free(PeerReduce *pr) {
  if (pr->bases_dev) cudaFree(pr->bases_dev);
  if (pr->step_dev) cudaFree(pr->step_dev);
  pr->bases_dev = nullptr;
  pr->step_dev = nullptr;
  pr->world = 0;
}

// the sum over all ranks replaces `grads` (n floats); stream-ordered, may be captured
int peer_reduce_run(b200_ctx *ctx, const PeerReduce *pr, float *grads) {
  B200_REQUIRE(pr->world >= 2 && pr->bases_dev && pr->step_dev, "peer_reduce_run: not initialised");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(grads) & 15) == 0, "peer_reduce_run: unaligned bucket");
  PeerArgs a;
  a.grads = grads;
  a.bases = pr->bases_dev;
  a.step = pr->step_dev;
  a.err = ctx->dev_err;
  a.rank = pr->rank;
  a.world = pr->world;
  a.n = pr->n;
  a.npad = pr_npad(pr->n);
  a.chunk = (pr->n + PR_CHUNKS - 1) / PR_CHUNKS;
  a.chunk = (a.chunk + 3) / 4 * 4;
  peer_reduce_kernel<<<PR_CHUNKS, PR_THREADS, 0, ctx->stream>>>(a);
  B200_LAUNCHED();
  peer_advance_kernel<<<1, 1, 0, ctx->stream>>>(pr->step_dev);
  B200_LAUNCHED();
  return 0;
}

}  // namespace b200
