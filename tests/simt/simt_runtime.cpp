/* Fiber scheduler of the SIMT emulator (see include/simt_emul.h). */
#include "simt_emul.h"

namespace simt {
Fiber *cur = nullptr;
ucontext_t sched;
simt_dim3 block_idx, grid_dim, block_dim;
unsigned live_threads = 0;
unsigned cta_count = 0, cta_gen = 0;
unsigned warp_count[64], warp_gen[64];
unsigned long long warp_slot[64][32];

static Body g_body;
static void *g_arg;

static void trampoline() {
  g_body(g_arg);
  cur->done = 1;
  swapcontext(&cur->ctx, &sched);
}

void run_grid(Body body, void *arg, simt_dim3 grid, simt_dim3 block) {
  const unsigned nthreads = block.x * block.y * block.z;
  const size_t stack_size = 256 * 1024;
  Fiber *fibers = (Fiber *)calloc(nthreads, sizeof(Fiber));
  for (unsigned t = 0; t < nthreads; t++) fibers[t].stack = (char *)malloc(stack_size);
  g_body = body;
  g_arg = arg;
  grid_dim = grid;
  block_dim = block;
  for (unsigned bz = 0; bz < grid.z; bz++)
    for (unsigned by = 0; by < grid.y; by++)
      for (unsigned bx = 0; bx < grid.x; bx++) {
        block_idx = simt_dim3{bx, by, bz};
        live_threads = nthreads;
        cta_count = 0;
        memset(warp_count, 0, sizeof(warp_count));
        for (unsigned t = 0; t < nthreads; t++) {
          Fiber &f = fibers[t];
          f.done = 0;
          f.linear = t;
          f.tid = simt_dim3{t % block.x, (t / block.x) % block.y, t / (block.x * block.y)};
          getcontext(&f.ctx);
          f.ctx.uc_stack.ss_sp = f.stack;
          f.ctx.uc_stack.ss_size = stack_size;
          f.ctx.uc_link = &sched;
          makecontext(&f.ctx, trampoline, 0);
        }
        unsigned remaining = nthreads;
        while (remaining) {
          for (unsigned t = 0; t < nthreads; t++) {
            if (fibers[t].done) continue;
            cur = &fibers[t];
            swapcontext(&sched, &cur->ctx);
            if (fibers[t].done == 1) {
              fibers[t].done = 2;
              remaining--;
            }
          }
        }
      }
  for (unsigned t = 0; t < nthreads; t++) free(fibers[t].stack);
  free(fibers);
}
}  // namespace simt
