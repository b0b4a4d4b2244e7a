// Host-side schedule evaluator used by the planner's search loop (hundreds of thousands of
// candidate evaluations for large graphs).  Same model as PipeGraph.simulate in
// parallel/pipe_graph.py, which stays the oracle: every rank runs its work list in order, a work
// item starts once its inputs have arrived, and every directed rank pair is a serial FIFO
// channel whose transfers take the edge's send time.
#include <algorithm>
#include <cstdint>
#include <vector>

extern "C" __attribute__((visibility("default")))
double pf_sim_schedule(int n_rank, int n_stage, int batch_cnt, const double* fwd_ms,
                       const double* bwd_ms, const double* optim_ms, const int* stage_rank,
                       int n_edge, const int* e_src, const int* e_dst, const double* e_ms,
                       const int* work_off, const int* work_stage, const int* work_mb,
                       const uint8_t* work_fwd, double* rank_busy_out) {
  const double NONE = -1.0;
  std::vector<std::vector<int>> prod(n_stage), cons(n_stage);
  for (int e = 0; e < n_edge; ++e) {
    prod[e_dst[e]].push_back(e);
    cons[e_src[e]].push_back(e);
  }
  // arrival[(is_grad, edge, mb)]
  std::vector<double> arrive(2 * (size_t)n_edge * batch_cnt, NONE);
  auto aidx = [&](int grad, int e, int b) { return ((size_t)grad * n_edge + e) * batch_cnt + b; };
  std::vector<uint8_t> f_done((size_t)n_stage * batch_cnt, 0);
  std::vector<double> chan((size_t)n_rank * n_rank, 0.0);
  std::vector<int> ptr(n_rank);
  std::vector<double> now(n_rank, 0.0), busy(n_rank, 0.0);
  for (int r = 0; r < n_rank; ++r) ptr[r] = work_off[r];
  long remaining = work_off[n_rank] - work_off[0];
  while (remaining > 0) {
    bool progressed = false;
    for (int r = 0; r < n_rank; ++r) {
      while (ptr[r] < work_off[r + 1]) {
        const int s = work_stage[ptr[r]], b = work_mb[ptr[r]];
        const bool fwd = work_fwd[ptr[r]] != 0;
        double t0 = now[r];
        bool ok = true;
        if (fwd) {
          for (int e : prod[s]) {
            const double a = arrive[aidx(0, e, b)];
            if (a == NONE) { ok = false; break; }
            t0 = std::max(t0, a);
          }
        } else {
          if (!f_done[(size_t)s * batch_cnt + b]) ok = false;
          for (int e : cons[s]) {
            if (!ok) break;
            const double a = arrive[aidx(1, e, b)];
            if (a == NONE) { ok = false; break; }
            t0 = std::max(t0, a);
          }
        }
        if (!ok) break;
        const double dur = fwd ? fwd_ms[s] : bwd_ms[s];
        const double t1 = t0 + dur;
        busy[r] += dur;
        now[r] = t1;
        if (fwd) f_done[(size_t)s * batch_cnt + b] = 1;
        const std::vector<int>& outs = fwd ? cons[s] : prod[s];
        for (int e : outs) {
          const int other = fwd ? e_dst[e] : e_src[e];
          const int r2 = stage_rank[other];
          double t = t1;
          if (r2 != r) {
            double& c = chan[(size_t)r * n_rank + r2];
            t = std::max(t1, c) + e_ms[e];
            c = t;
          }
          arrive[aidx(fwd ? 0 : 1, e, b)] = t;
        }
        ++ptr[r];
        --remaining;
        progressed = true;
      }
    }
    if (!progressed) return -1.0;   // deadlock: an input is never produced
  }
  double span = 0.0;
  for (int r = 0; r < n_rank; ++r) {
    span = std::max(span, now[r] + optim_ms[r]);
    if (rank_busy_out) rank_busy_out[r] = busy[r];
  }
  return span;
}
