// Oracle (test infrastructure): fork-join pool and the row-parallel
// matrix-vector / batched products. Restates crates/aot-kernels/src/pool.rs and
// crates/aot-kernels/src/matvec.rs:300-583. Thread count and chunking change
// who computes a row, never its value.
#include <immintrin.h>
#include <sched.h>
#include <time.h>

#include <atomic>
#include <functional>
#include <thread>
#include <vector>

#include "oracle_internal.h"

struct orc_pool {
  int n_threads = 1;
  std::atomic<size_t> epoch{0};
  std::atomic<int> pending{0};
  std::atomic<bool> stop{false};
  const std::function<void(int, int)>* job = nullptr;
  std::vector<std::thread> workers;
};

// pool.rs:120-149: spin, then yield, then sleep 200 us while idle.
static void worker_main(orc_pool* p, int tid) {
  size_t seen = 0;
  for (;;) {
    unsigned spins = 0;
    for (;;) {
      size_t e = p->epoch.load(std::memory_order_acquire);
      if (e != seen) {
        seen = e;
        break;
      }
      if (p->stop.load(std::memory_order_relaxed)) return;
      spins++;
      if (spins < 50000) {
        _mm_pause();
      } else if (spins < 60000) {
        sched_yield();
      } else {
        struct timespec ts = {0, 200000};
        nanosleep(&ts, nullptr);
      }
    }
    (*p->job)(tid, p->n_threads);
    p->pending.fetch_sub(1, std::memory_order_acq_rel);
  }
}

// pool.rs:66-83
void orc_pool_run(orc_pool* p, const std::function<void(int, int)>& f) {
  int n = p->n_threads;
  if (n == 1) {
    f(0, 1);
    return;
  }
  p->job = &f;
  p->pending.store(n - 1, std::memory_order_relaxed);
  p->epoch.fetch_add(1, std::memory_order_release);
  f(0, n);
  while (p->pending.load(std::memory_order_acquire) != 0) _mm_pause();
}

// pool.rs:91-108: chunks handed out by an atomic counter.
void orc_pool_run_chunks(orc_pool* p, size_t n, size_t chunk, const std::function<void(size_t, size_t)>& f) {
  if (chunk < 1) chunk = 1;
  if (n == 0) return;
  if (p->n_threads == 1 || n <= chunk) {
    f(0, n);
    return;
  }
  std::atomic<size_t> next{0};
  orc_pool_run(p, [&](int, int) {
    for (;;) {
      size_t start = next.fetch_add(chunk, std::memory_order_relaxed);
      if (start >= n) break;
      size_t end = start + chunk < n ? start + chunk : n;
      f(start, end);
    }
  });
}

// matvec.rs:316-318
static size_t row_chunk(size_t rows, int nth) {
  size_t c = rows / ((size_t)nth * 8);
  return c < 8 ? 8 : c;
}

extern "C" {

orc_pool* orc_pool_new(int n_threads) {
  orc_pool* p = new orc_pool();
  p->n_threads = n_threads < 1 ? 1 : n_threads;
  for (int t = 1; t < p->n_threads; t++) p->workers.emplace_back(worker_main, p, t);
  return p;
}

void orc_pool_free(orc_pool* p) {
  if (!p) return;
  p->stop.store(true, std::memory_order_release);
  for (auto& w : p->workers) w.join();
  delete p;
}

int orc_pool_threads(const orc_pool* p) { return p->n_threads; }

// matvec.rs:300-311
void orc_matvec(orc_pool* p, int table, int kind, float* out, const uint8_t* w, const void* x, size_t rows,
                size_t cols) {
  orc_dot_fn dot = orc_get_dot(table, kind);
  size_t rb = orc_row_bytes(kind, cols);
  orc_pool_run_chunks(p, rows, row_chunk(rows, p->n_threads), [&](size_t a, size_t b) {
    for (size_t r = a; r < b; r++) out[r] = dot(w + r * rb, x, cols);
  });
}

// matvec.rs:407-439
void orc_matvec2(orc_pool* p, int table, int kind, float* out_a, float* out_b, const uint8_t* w_a,
                 const uint8_t* w_b, const void* x, size_t rows, size_t cols) {
  orc_dot_fn dot = orc_get_dot(table, kind);
  size_t rb = orc_row_bytes(kind, cols);
  orc_pool_run_chunks(p, rows, row_chunk(rows, p->n_threads), [&](size_t a, size_t b) {
    for (size_t r = a; r < b; r++) {
      out_a[r] = dot(w_a + r * rb, x, cols);
      out_b[r] = dot(w_b + r * rb, x, cols);
    }
  });
}

// matvec.rs:323-343: one region over the concatenated q/k/v row space.
void orc_matvec3(orc_pool* p, int table, int kind, float* o0, float* o1, float* o2, const uint8_t* w0,
                 const uint8_t* w1, const uint8_t* w2, const void* x, size_t r0, size_t r1, size_t r2,
                 size_t cols) {
  orc_dot_fn dot = orc_get_dot(table, kind);
  size_t rb = orc_row_bytes(kind, cols);
  size_t total = r0 + r1 + r2;
  orc_pool_run_chunks(p, total, row_chunk(total, p->n_threads), [&](size_t a, size_t b) {
    for (size_t r = a; r < b; r++) {
      if (r < r0) {
        o0[r] = dot(w0 + r * rb, x, cols);
      } else if (r < r0 + r1) {
        o1[r - r0] = dot(w1 + (r - r0) * rb, x, cols);
      } else {
        o2[r - r0 - r1] = dot(w2 + (r - r0 - r1) * rb, x, cols);
      }
    }
  });
}

// matvec.rs:479-522: 8-row blocks, four tokens at a time through the 1x4
// micro-kernel when the table has one, token-major output.
void orc_matmul(orc_pool* p, int table, int kind, float* out, const uint8_t* w, const void* xs, size_t m,
                size_t rows, size_t cols) {
  orc_dot_fn dot = orc_get_dot(table, kind);
  orc_dot4_fn dot4 = orc_get_dot4(table, kind);
  size_t rb = orc_row_bytes(kind, cols);
  int act = orc_activation(kind);
  // Bytes of one token's activation vector.
  size_t xstride = act == ORC_ACT_Q8_K ? cols / 256 * sizeof(orc_block_q8_k)
                   : act == ORC_ACT_Q8_0 ? cols / 32 * sizeof(orc_block_q8_0)
                                         : cols * sizeof(float);
  const uint8_t* xb = (const uint8_t*)xs;
  const size_t RB = 8;
  size_t chunk = rows / ((size_t)p->n_threads * 4);
  if (chunk < RB) chunk = RB;
  chunk = (chunk + RB - 1) / RB * RB;
  orc_pool_run_chunks(p, rows, chunk, [&](size_t a, size_t b) {
    for (size_t r0 = a; r0 < b;) {
      size_t r1 = r0 + RB < b ? r0 + RB : b;
      size_t i = 0;
      if (dot4) {
        for (; i + 4 <= m; i += 4) {
          const void* x4[4] = {xb + i * xstride, xb + (i + 1) * xstride, xb + (i + 2) * xstride,
                               xb + (i + 3) * xstride};
          for (size_t r = r0; r < r1; r++) {
            float v[4];
            dot4(w + r * rb, x4, cols, v);
            for (int k = 0; k < 4; k++) out[(i + k) * rows + r] = v[k];
          }
        }
      }
      for (; i < m; i++) {
        for (size_t r = r0; r < r1; r++) out[i * rows + r] = dot(w + r * rb, xb + i * xstride, cols);
      }
      r0 = r1;
    }
  });
}

}  // extern "C"
