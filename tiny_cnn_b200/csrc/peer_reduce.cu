// Sum of the gradient bucket over the replicas of a data-parallel job, through peer memory
// (NVLink / NVSwitch), as kernels that are recorded in the CUDA graph of a step.
// It is the device form of what the data-parallel driver otherwise does with one NCCL all-reduce
// between two graphs: edge::merge_grads over all replicas (tiny_dnn/network.h:880-906 sums the
// per-sample gradients of ONE mini-batch; replicas extend that sum across GPUs, with no 1/N).
//
// Every rank owns a buffer that all ranks have mapped ("symmetric" memory):
//   slots[2][world][npad] floats, then flags[2][2][PR_CHUNKS] counters, then words[2][world][ll_n]
//   8-byte words (only when the late region is small, see below)
// A step uses the half `step & 1`.  The bucket has two regions:
//   early = [split, n)  gradients that are final long before the backward pass ends (every layer
//                       but the first one with parameters); pushed from a side branch of the step
//                       as soon as they exist, so their trip over NVLink hides under the rest
//   late  = [0, split)  the first layer's gradients, pushed by the kernel that sums
// PUSH (peer_push_kernel): block b copies chunk b of a region from the local bucket into slot
// [rank] of EVERY rank's buffer (plain peer stores), makes the stores visible (system fence) and
// adds 1 to flag [half][region][b] of every rank.  It waits for nothing.
// SUM (peer_sum_kernel): block b first pushes late chunk b (unless told the push was done), then
// waits until its own flags [half][early][b] and [half][late][b] have received `world`
// additions for this use of the half, then adds the `world` slots of both chunks in rank order --
// the same order on every rank, so the replicas stay bit-identical -- into the local bucket.
// No block waits for another block of its own GPU.  Every wait is bounded by wall time: a block
// whose wait runs out sets the context's error word (code 7) and leaves its chunks unsummed; the
// optimizer kernel that follows reads that word and changes nothing, so a rank that timed out keeps
// its parameters of the step before.  The other ranks may have completed the step: after a timeout
// the replicas differ and the flag counters are out of step, which is terminal for this group of
// ranks (restart from a checkpoint).  A half is reused only two steps later, after every rank has
// passed the step in between.  Every load is CTA-local or a plain load of this GPU's own memory;
// the peers are only written.
// A SMALL late region (at most PR_LL_MAX floats -- the first layer of a convolutional net) travels as
// flagged words instead: every float is stored to the peers as ONE aligned 8-byte scalar
// {value, step + 1}, which arrives whole, and the summing thread polls the word in its own memory
// until the flag is this step's.  No fence, no counter, no second trip over NVLink: the late
// region sits on the critical path of the step (it leaves when the backward pass has ended), and
// store -> fence -> counter -> poll costs three NVLink traversals where this costs one.
#include "common.cuh"
#include "device_utils.cuh"

namespace b200 {

namespace {

constexpr int PR_CHUNKS = 128;   // blocks: all resident at once on 148 SMs
constexpr int PR_THREADS = 256;
constexpr long long PR_LL_MAX = 65536;  // floats: above this, bandwidth matters more than latency

// one float and the flag of its step as a single 8-byte scalar store / load: single-copy atomic
__device__ __forceinline__ void st_word_sys(unsigned long long *dst, float v, unsigned flag) {
  const unsigned long long w = ((unsigned long long)flag << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;\n" ::"l"(dst), "l"(w) : "memory");
}
__device__ __forceinline__ bool ld_word_sys(const unsigned long long *src, unsigned flag, float *v) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];\n" : "=l"(w) : "l"(src) : "memory");
  *v = __uint_as_float((unsigned)(w & 0xffffffffull));
  return (unsigned)(w >> 32) == flag;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerArgs {
  float *grads;              // local bucket, n floats: read, then overwritten with the sum
  float *const *bases;       // [world] base of every rank's buffer as mapped here
  unsigned *step;            // [0] number of reductions done so far, [1] blocks of the summing kernel that ended
  int *err;
  int rank, world;
  long long n, npad;         // floats; npad is a multiple of 4
  long long lo[2], chunk[2]; // region r = [lo[r], hi[r]) cut into PR_CHUNKS chunks of chunk[r] floats
  long long hi[2];           // lo, chunk multiples of 4
  long long ll_n;            // words per rank and half of the flagged-word area; 0 = the late region uses slots + counters
  unsigned long long timeout_ns;
};

// copy [c0, c1) of the local bucket into slot `slot_off` of every rank's buffer
__device__ __forceinline__ void push_range(const PeerArgs &a, size_t slot_off, long long c0, long long c1) {
  const int tid = threadIdx.x;
  for (long long i = c0 + 4 * tid; i < c1; i += 4 * PR_THREADS) {
    if (i + 4 <= c1) {
      const float4 v = *reinterpret_cast<const float4 *>(a.grads + i);
      for (int p = 0; p < a.world; ++p) *reinterpret_cast<float4 *>(a.bases[p] + slot_off + i) = v;
    } else {
      for (long long j = i; j < c1; ++j) {
        const float v = a.grads[j];
        for (int p = 0; p < a.world; ++p) a.bases[p][slot_off + j] = v;
      }
    }
  }
}

__device__ __forceinline__ void chunk_range(const PeerArgs &a, int region, int b, long long *c0, long long *c1) {
  long long s = a.lo[region] + (long long)b * a.chunk[region];
  long long e = s + a.chunk[region];
  if (e > a.hi[region]) e = a.hi[region];
  if (s > e) s = e;
  *c0 = s;
  *c1 = e;
}

// push one region's chunk and signal; all threads of the block call it
__device__ __forceinline__ void push_and_signal(const PeerArgs &a, int region, int half, int b) {
  long long c0, c1;
  chunk_range(a, region, b, &c0, &c1);
  if (c0 >= c1) return;  // an empty chunk is neither signalled nor waited for (same on every rank)
  const size_t flag_off = (size_t)2 * a.world * a.npad;  // floats before the flags
  const size_t my_slot = ((size_t)half * a.world + a.rank) * a.npad;
  push_range(a, my_slot, c0, c1);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world) {
    unsigned *flag = reinterpret_cast<unsigned *>(a.bases[threadIdx.x] + flag_off) + (half * 2 + region) * PR_CHUNKS + b;
    __threadfence_system();  // the signalling thread orders the block's stores (seen through the barrier) before the flag
    atomicAdd_system(flag, 1u);
  }
}

// the flagged-word area of rank p's buffer: words[half][source rank][ll_n]
__device__ __forceinline__ unsigned long long *words_of(const PeerArgs &a, int p, int half, int src) {
  const size_t before = ((size_t)2 * a.world * a.npad + (size_t)4 * PR_CHUNKS) * sizeof(float);  // bytes, a multiple of 16
  return reinterpret_cast<unsigned long long *>(reinterpret_cast<char *>(a.bases[p]) + before) +
         ((size_t)half * a.world + src) * a.ll_n;
}

// late chunk b as flagged words into every other rank's buffer; waits for nothing, signals nothing
__device__ __forceinline__ void push_words(const PeerArgs &a, int half, unsigned flag, int b) {
  long long c0, c1;
  chunk_range(a, 0, b, &c0, &c1);
  for (long long i = c0 + threadIdx.x; i < c1; i += PR_THREADS) {
    const float v = a.grads[i];
    for (int p = 0; p < a.world; ++p)
      if (p != a.rank) st_word_sys(words_of(a, p, half, a.rank) + i, v, flag);
  }
}

// regions: bit 0 = late [0, split), bit 1 = early [split, n)
__global__ void __launch_bounds__(PR_THREADS) peer_push_kernel(const PeerArgs a, int regions) {
  const int b = blockIdx.x;
  const unsigned step = *a.step;
  const int half = (int)(step & 1u);
  if (regions & 2) push_and_signal(a, 1, half, b);
  if (regions & 1) {
    if (a.ll_n) push_words(a, half, step + 1u, b);
    else push_and_signal(a, 0, half, b);
  }
}

// the last block of the summing kernel to end closes this use of the buffer half: every block has
// read the step number by then
__device__ __forceinline__ void sum_block_done(const PeerArgs &a) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.step + 1, 1u) == gridDim.x - 1) {
      a.step[1] = 0u;
      __threadfence();
      a.step[0] += 1u;
    }
  }
}

// regions: bit 0 = late, bit 1 = early -- the regions this launch waits for and sums; `advance`: this
// launch is the last one of the step that uses the buffer half
__global__ void __launch_bounds__(PR_THREADS) peer_sum_kernel(const PeerArgs a, int push_late, int regions,
                                                              int advance) {
  __shared__ int s_fail;
  const int tid = threadIdx.x, b = blockIdx.x;
  const unsigned step = *a.step;
  const int half = (int)(step & 1u);
  const unsigned target = (step / 2u + 1u) * (unsigned)a.world;  // additions a flag has seen after this use
  const size_t flag_off = (size_t)2 * a.world * a.npad;
  const bool words = a.ll_n != 0;  // the late region travels as flagged words
  if (push_late) {
    if (words) push_words(a, half, step + 1u, b);
    else push_and_signal(a, 0, half, b);
  }
  long long c0[2], c1[2];
  chunk_range(a, 0, b, &c0[0], &c1[0]);
  chunk_range(a, 1, b, &c0[1], &c1[1]);
  // wait for every rank's chunks (bounded by wall time)
  if (tid == 0) {
    const unsigned *flags = reinterpret_cast<const unsigned *>(a.bases[a.rank] + flag_off) + half * 2 * PR_CHUNKS + b;
    int fail = 0;
    unsigned long long t0 = 0, t1;
    for (int region = 0; region < 2 && !fail; ++region) {
      if (!(regions >> region & 1) || c0[region] >= c1[region] || (region == 0 && words)) continue;
      const unsigned *mine = flags + region * PR_CHUNKS;
      if (ld_acquire_sys(mine) >= target) continue;
      if (!t0) asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
      for (;;) {
        bool done = false;
        for (int k = 0; k < 64 && !done; ++k) done = ld_acquire_sys(mine) >= target;
        if (done) break;
        asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1));
        if (t1 - t0 > a.timeout_ns) {
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
    if (advance) sum_block_done(a);
    return;
  }
  // sum the slots in rank order; the peers' stores sit in this GPU's memory / L2, not in this SM's L1
  const float *slots = a.bases[a.rank] + (size_t)half * a.world * a.npad;
  if (words && (regions & 1)) {
    // every thread polls the words of its own floats, rank by rank: the sum keeps the rank order
    const unsigned flag = step + 1u;
    unsigned long long t0 = 0, t1;
    bool fail = false;
    for (long long i = c0[0] + tid; i < c1[0] && !fail; i += PR_THREADS) {
      float sum = 0.f;
      for (int r = 0; r < a.world && !fail; ++r) {
        float v;
        if (r == a.rank) {
          v = a.grads[i];
        } else {
          const unsigned long long *w = words_of(a, a.rank, half, r) + i;
          while (!ld_word_sys(w, flag, &v)) {
            bool done = false;
            for (int k = 0; k < 64 && !done; ++k) done = ld_word_sys(w, flag, &v);
            if (done) break;
            if (!t0) asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1));
            if (t1 - t0 > a.timeout_ns) {
              fail = true;
              break;
            }
          }
        }
        sum = r == 0 ? v : __fadd_rn(sum, v);
      }
      if (!fail) a.grads[i] = sum;
    }
    if (fail && a.err) atomicExch(a.err, 7);
  }
  for (int region = words ? 1 : 0; region < 2; ++region) {
    if (!(regions >> region & 1)) continue;
    for (long long i = c0[region] + 4 * tid; i < c1[region]; i += 4 * PR_THREADS) {
      if (i + 4 <= c1[region]) {
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
        for (long long j = i; j < c1[region]; ++j) {
          float s = __ldcg(slots + j);
          for (int r = 1; r < a.world; ++r) s = __fadd_rn(s, __ldcg(slots + (size_t)r * a.npad + j));
          a.grads[j] = s;
        }
      }
    }
  }
  if (advance) sum_block_done(a);
}

long long pr_npad(long long n) { return (n + 3) / 4 * 4; }

PeerArgs make_args(b200_ctx *ctx, const PeerReduce *pr, float *grads) {
  PeerArgs a;
  a.grads = grads;
  a.bases = pr->bases_dev;
  a.step = pr->step_dev;
  a.err = ctx->dev_err;
  a.rank = pr->rank;
  a.world = pr->world;
  a.n = pr->n;
  a.npad = pr_npad(pr->n);
  a.lo[0] = 0;
  a.hi[0] = pr->split;
  a.lo[1] = pr->split;
  a.hi[1] = pr->n;
  for (int r = 0; r < 2; ++r) {
    long long len = a.hi[r] - a.lo[r];
    long long c = (len + PR_CHUNKS - 1) / PR_CHUNKS;
    a.chunk[r] = (c + 3) / 4 * 4;
  }
  a.ll_n = pr->ll_n;
  a.timeout_ns = pr->timeout_ns;
  return a;
}

int check_run(const PeerReduce *pr, const float *grads) {
  B200_REQUIRE(pr->world >= 2 && pr->bases_dev && pr->step_dev, "peer reduce: not initialised");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(grads) & 15) == 0, "peer reduce: unaligned bucket");
  return 0;
}

}  // namespace

// bytes of the buffer every rank must provide (zero-filled, mapped by all ranks)
long long peer_reduce_words(long long split) { return split > 0 && split <= PR_LL_MAX ? pr_npad(split) : 0; }

size_t peer_reduce_bytes(long long n, long long split, int world) {
  return ((size_t)2 * world * pr_npad(n)) * sizeof(float) + (size_t)4 * PR_CHUNKS * sizeof(unsigned) +
         (size_t)2 * world * peer_reduce_words(split) * sizeof(unsigned long long);
}

int peer_reduce_init(b200_ctx *ctx, PeerReduce *pr, long long n, long long split, int rank, int world,
                     const unsigned long long *bases, int timeout_ms) {
  B200_REQUIRE(world >= 2 && world <= PR_THREADS && rank >= 0 && rank < world && n > 0 && bases,
               "peer_reduce_init: bad argument");
  B200_REQUIRE(split >= 0 && split <= n && (split % 4 == 0 || split == n),
               "peer_reduce_init: split %lld outside 0..%lld or not a multiple of 4", split, n);
  B200_REQUIRE(timeout_ms >= 0, "peer_reduce_init: negative time limit");
  for (int p = 0; p < world; ++p)
    B200_REQUIRE(bases[p] != 0 && (bases[p] & 15) == 0, "peer_reduce_init: buffer of rank %d is NULL or unaligned", p);
  peer_reduce_free(pr);
  pr->rank = rank;
  pr->world = world;
  pr->n = n;
  pr->split = split;
  pr->ll_n = peer_reduce_words(split);
  if (const char *e = getenv("B200_PEER_WORDS"))
    if (atoi(e) == 0) pr->ll_n = 0;  // the buffer has room for the words either way
  pr->timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1000000ull;
  B200_CUDA(cudaMalloc(&pr->bases_dev, sizeof(float *) * world));
  B200_CUDA(cudaMemcpy(pr->bases_dev, bases, sizeof(float *) * world, cudaMemcpyHostToDevice));
  B200_CUDA(cudaMalloc(&pr->step_dev, 2 * sizeof(unsigned)));
  B200_CUDA(cudaMemset(pr->step_dev, 0, 2 * sizeof(unsigned)));
  (void)ctx;
  // these kernels run beside the persistent tensor-core kernels, which hold the largest shared-memory
  // carve-out of an SM; asking for the same carve-out keeps an SM from being reconfigured between them
  const char *co = getenv("B200_PEER_CARVEOUT");
  if (!co || atoi(co) != 0) {
    cudaFuncSetAttribute(peer_push_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(peer_sum_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  }
  return 0;
}

void peer_reduce_free(PeerReduce *pr) {
  if (pr->bases_dev) cudaFree(pr->bases_dev);
  if (pr->step_dev) cudaFree(pr->step_dev);
  pr->bases_dev = nullptr;
  pr->step_dev = nullptr;
  pr->world = 0;
}

// push the early region [split, n) of `grads` to every rank; waits for nothing
int peer_reduce_push_early(b200_ctx *ctx, const PeerReduce *pr, float *grads) {
  B200_TRY(check_run(pr, grads));
  if (pr->split >= pr->n) return 0;
  peer_push_kernel<<<PR_CHUNKS, PR_THREADS, 0, ctx->stream>>>(make_args(ctx, pr, grads), 2);
  B200_LAUNCHED();
  return 0;
}

// push both regions; waits for nothing (a rank's whole contribution, for callers that run the
// ranks of one GPU one after the other)
int peer_reduce_push_all(b200_ctx *ctx, const PeerReduce *pr, float *grads) {
  B200_TRY(check_run(pr, grads));
  peer_push_kernel<<<PR_CHUNKS, PR_THREADS, 0, ctx->stream>>>(make_args(ctx, pr, grads), 3);
  B200_LAUNCHED();
  return 0;
}

// wait for every rank's early region and sum it, on the stream the early push went to: by the end of
// the backward pass only the late region is left.  Does not end the use of the buffer half.
int peer_reduce_sum_early(b200_ctx *ctx, const PeerReduce *pr, float *grads) {
  B200_TRY(check_run(pr, grads));
  if (pr->split >= pr->n) return 0;
  peer_sum_kernel<<<PR_CHUNKS, PR_THREADS, 0, ctx->stream>>>(make_args(ctx, pr, grads), 0, 2, 0);
  B200_LAUNCHED();
  return 0;
}

// (push the late region unless `late_pushed`,) wait for every rank's regions -- the late one only when
// `early_summed` -- and replace `grads` by the sum over the ranks; ends this use of the buffer half
int peer_reduce_finish(b200_ctx *ctx, const PeerReduce *pr, float *grads, int late_pushed, int early_summed) {
  B200_TRY(check_run(pr, grads));
  peer_sum_kernel<<<PR_CHUNKS, PR_THREADS, 0, ctx->stream>>>(make_args(ctx, pr, grads), late_pushed ? 0 : 1,
                                                            early_summed ? 1 : 3, 1);
  B200_LAUNCHED();
  return 0;
}

// the whole reduction on one stream: early push, then late push + wait + sum
int peer_reduce_run(b200_ctx *ctx, const PeerReduce *pr, float *grads) {
  B200_TRY(peer_reduce_push_early(ctx, pr, grads));
  return peer_reduce_finish(ctx, pr, grads, 0, 0);
}

}  // namespace b200
