/* Combination of per-GPU partial results through peer memory: what follows a
 * reduction whose reduced extent is sharded over the GPUs of a communicator
 * (GpuReduction_call_sharded). One launch per GPU replaces the all-reduce the
 * reference's collectives would be asked for
 * (src/gpuarray_collectives_cuda_nccl.c:286-316) and, for (value, index)
 * operators - for which those collectives have no operator at all (:158-185) -
 * two all-reduces and the kernels between them.
 *
 * Every GPU owns a WINDOW of device memory that all peers of the communicator
 * have mapped (ga_comm.c):
 *
 *     flags  [2][GA_XC_MAX_RANKS][GA_XC_MAX_CTAS]  unsigned long long
 *     data   at GA_XC_DATA_OFF: [2][nranks] slots of slot_bytes
 *            a slot: n values, then at idx_off n indices (pair kernels only)
 *
 * Exchange number `seq` (1, 2, ... in the order of the calls, the same on all
 * ranks) uses half seq & 1 of both. CTA c of rank r owns outputs
 * [c * chunk, (c + 1) * chunk):
 *   push     stores its partials into slot [seq & 1][r] of EVERY peer's window
 *            (plain stores over NVLink), makes them visible system-wide, then
 *            sets flag [seq & 1][r][c] = seq in every peer's window;
 *   combine  waits until its OWN window's flags [seq & 1][p][c] reach seq for
 *            every peer p, then folds its own partial and the peers' slots
 *            in rank order 0, 1, ... (every rank computes the same bits) and
 *            writes the result over its partial.
 * Two halves suffice: a peer can only start exchange seq + 2 (the next user of
 * the same half) after it finished seq + 1, which needed this rank's flag of
 * seq + 1, which this rank sets after its kernel of seq has completed.
 *
 * Every wait is bounded: a peer that does not show up within timeout_ns makes
 * the CTA record 1 in *status (host-visible) and carry on with whatever the
 * slots hold; the host refuses further exchanges on that communicator.
 * The kernels of one exchange run on DIFFERENT GPUs, one process per GPU;
 * nothing here waits for another launch on the same GPU.
 *
 * Defines:
 *   GA_XC_T        element type of the partial values
 *   GA_XC_PAIR     0: accumulating operator; 1: (value, index) operator;
 *                  2: value-only minimum / maximum whose ties (+0.0 against
 *                  -0.0) go to the rank with the lower `key` - the shard's
 *                  first coordinate when the sharded axis is the slowest
 *                  reduced one, so that the earlier element wins as on one
 *                  GPU. The key travels in the first index cell of the slot.
 *   GA_XC_MIN      pair kernels: 1 minimum, 0 maximum
 *   GA_XC_W_T      pair kernels: type the comparison runs in; accumulating
 *                  kernels: type the fold runs in (float for ga_half)
 *   GA_XC_LOAD(x)  GA_XC_T -> GA_XC_W_T,  GA_XC_STORE(w)  GA_XC_W_T -> GA_XC_T
 *   GA_XC_OP(a,b)  accumulating kernels: the fold of two GA_XC_W_T
 */
#include "cluda.h"

#define GA_XC_MAX_RANKS 16
#define GA_XC_MAX_CTAS 64
#define GA_XC_DATA_OFF 32768
#define GA_XC_THREADS 256
#define GA_XC_NONE 0xFFFFFFFFFFFFFFFFULL

#ifndef SIMT_EMUL_H
/* ga__fence_system + ga__st_release_sys publish data written to a peer;
 * ga__ld_acquire_sys polls a flag a peer writes; ga__ld_volatile reads what a
 * peer wrote without taking a line from this SM's L1 (a peer's stores arrive in
 * the L2 of the GPU that owns the memory, not in its L1s). */
static __device__ __forceinline__ void ga__fence_system() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
static __device__ __forceinline__ void ga__st_release_sys(unsigned long long *p,
                                                          unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
static __device__ __forceinline__ unsigned long long ga__ld_acquire_sys(
    const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
static __device__ __forceinline__ unsigned long long ga__globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
static __device__ __forceinline__ void ga__nanosleep(unsigned int ns) {
  asm volatile("nanosleep.u32 %0;" ::"r"(ns));
}
template <int BYTES> struct ga__raw_of;
template <> struct ga__raw_of<1> { typedef unsigned char t; };
template <> struct ga__raw_of<2> { typedef unsigned short t; };
template <> struct ga__raw_of<4> { typedef unsigned int t; };
template <> struct ga__raw_of<8> { typedef unsigned long long t; };
template <typename T>
static __device__ __forceinline__ T ga__ld_volatile(const T *p) {
  typedef typename ga__raw_of<sizeof(T)>::t raw_t;
  const raw_t r = *reinterpret_cast<const volatile raw_t *>(p);
  return *reinterpret_cast<const T *>(&r);
}
#endif

struct ga__xc_layout {
  unsigned long long n;          /* outputs */
  unsigned long long seq;        /* number of this exchange on the communicator, from 1 */
  unsigned long long slot_bytes; /* one rank's slot in a data half */
  unsigned long long idx_off;    /* byte offset of the indices inside a slot */
  unsigned long long timeout_ns; /* longest wait for one peer */
  unsigned long long key;        /* GA_XC_PAIR == 2: this rank's tie-break key */
  unsigned long long win[GA_XC_MAX_RANKS]; /* every rank's window as mapped here */
  unsigned int nranks, rank;
  unsigned int chunk;            /* outputs per CTA */
  unsigned int phases;           /* bit 0 push, bit 1 combine; 3 except under test */
};

extern "C" __global__ void __launch_bounds__(GA_XC_THREADS)
ga_exchange(const __grid_constant__ ga__xc_layout L, GA_XC_T *val, unsigned long long *idx,
            unsigned int *status) {
  ga__grid_dependency_sync();
  const unsigned int half = (unsigned int)(L.seq & 1);
  const unsigned long long lo = (unsigned long long)blockIdx.x * L.chunk;
  const unsigned long long hi = lo + L.chunk < L.n ? lo + L.chunk : L.n;
  const unsigned long long data0 = GA_XC_DATA_OFF + (unsigned long long)half * L.nranks * L.slot_bytes;
  const unsigned long long flag0 = (unsigned long long)half * GA_XC_MAX_RANKS * GA_XC_MAX_CTAS;

  if (L.phases & 1) {
#if GA_XC_PAIR == 2
    if (threadIdx.x == 0) /* every CTA sends the key: its flag must cover it */
      for (unsigned int p = 0; p < L.nranks; p++)
        if (p != L.rank)
          *reinterpret_cast<unsigned long long *>(reinterpret_cast<char *>(L.win[p]) + data0 +
                                                  L.rank * L.slot_bytes + L.idx_off) = L.key;
#endif
    for (unsigned long long k = lo + threadIdx.x; k < hi; k += GA_XC_THREADS) {
      const GA_XC_T v = val[k];
#if GA_XC_PAIR == 1
      const unsigned long long i = idx[k];
#endif
      for (unsigned int r = 1; r < L.nranks; r++) {
        unsigned int p = L.rank + r; /* every rank starts with another peer */
        if (p >= L.nranks) p -= L.nranks;
        char *slot = reinterpret_cast<char *>(L.win[p]) + data0 + L.rank * L.slot_bytes;
        reinterpret_cast<GA_XC_T *>(slot)[k] = v;
#if GA_XC_PAIR == 1
        reinterpret_cast<unsigned long long *>(slot + L.idx_off)[k] = i;
#endif
      }
    }
    ga__fence_system();
    __syncthreads();
    if (threadIdx.x < L.nranks && threadIdx.x != L.rank) {
      unsigned long long *flags = reinterpret_cast<unsigned long long *>(L.win[threadIdx.x]);
      ga__st_release_sys(flags + flag0 + L.rank * GA_XC_MAX_CTAS + blockIdx.x, L.seq);
    }
  }
  if (!(L.phases & 2)) return;

  if (threadIdx.x < L.nranks && threadIdx.x != L.rank) {
    const unsigned long long *flag = reinterpret_cast<const unsigned long long *>(L.win[L.rank]) +
                                     flag0 + threadIdx.x * GA_XC_MAX_CTAS + blockIdx.x;
    const unsigned long long t0 = ga__globaltimer_ns();
    unsigned int polls = 0;
    while (ga__ld_acquire_sys(flag) < L.seq) {
      if (++polls < 64) continue; /* the usual wait is a few microseconds: poll flat out first */
      ga__nanosleep(200);
      if ((polls & 15) == 0 && (ga__globaltimer_ns() - t0 > L.timeout_ns || polls > 0x7FFFFFF0u)) {
        *reinterpret_cast<volatile unsigned int *>(status) = 1u; /* every writer stores the same value */
        break;
      }
    }
  }
  __syncthreads();

  const char *mine = reinterpret_cast<const char *>(L.win[L.rank]) + data0;
  for (unsigned long long k = lo + threadIdx.x; k < hi; k += GA_XC_THREADS) {
#if GA_XC_PAIR
    /* the candidate with the better value wins, the lower index among equal
     * values (+0.0 == -0.0: the earlier one, as on one GPU); a NaN is only ever
     * delivered by the shard holding element 0, where it is the answer; index
     * all-ones marks a shard without a candidate */
    GA_XC_T bv = val[k];
    unsigned long long bi = GA_XC_NONE;
    GA_XC_W_T bw = GA_XC_LOAD(bv);
    bool fixed = false;
    for (unsigned int r = 0; r < L.nranks; r++) {
      GA_XC_T v;
      unsigned long long i;
      if (r == L.rank) {
        v = val[k];
#if GA_XC_PAIR == 1
        i = idx[k];
#else
        i = L.key;
#endif
      } else {
        const char *slot = mine + r * L.slot_bytes;
        v = ga__ld_volatile(reinterpret_cast<const GA_XC_T *>(slot) + k);
#if GA_XC_PAIR == 1
        i = ga__ld_volatile(reinterpret_cast<const unsigned long long *>(slot + L.idx_off) + k);
#else
        i = ga__ld_volatile(reinterpret_cast<const unsigned long long *>(slot + L.idx_off));
#endif
      }
      if (i == GA_XC_NONE || fixed) continue;
      const GA_XC_W_T w = GA_XC_LOAD(v);
      bool take;
      if (bi == GA_XC_NONE || w != w) {
        take = true;
      } else {
#if GA_XC_MIN
        take = w < bw || (w == bw && i < bi);
#else
        take = w > bw || (w == bw && i < bi);
#endif
      }
      if (take) {
        bv = v;
        bw = w;
        bi = i;
        fixed = w != w;
      }
    }
    val[k] = bv;
#if GA_XC_PAIR == 1
    idx[k] = bi;
#endif
#else
    GA_XC_W_T acc;
    for (unsigned int r = 0; r < L.nranks; r++) {
      const GA_XC_T v = r == L.rank
                            ? val[k]
                            : ga__ld_volatile(reinterpret_cast<const GA_XC_T *>(mine + r * L.slot_bytes) + k);
      const GA_XC_W_T w = GA_XC_LOAD(v);
      if (r == 0) {
        acc = w;
      } else {
        const GA_XC_W_T a = acc, b = w;
        acc = GA_XC_OP(a, b);
      }
    }
    val[k] = GA_XC_STORE(acc);
#endif
  }
}
