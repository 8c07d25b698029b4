// C-ABI shim around the reference's own native CPU hard forward (test infrastructure only).
//
// Compiled from the reference sources where they lie (never copied into this repository):
//   dism_v3/python/flash_dism/inference/csrc/prefill.hpp  Builder (:426-515), finish (:517-599),
//   execute<T> (:603-625); planner.hpp  Planner::append / advance (:132-149, :253-310) for the longest match length.
// The build recipe is oracle/Makefile; the output goes to oracle/_ref/.
// One call plans and executes one (batch, head) sequence: labels -> Program -> output rows.
#include "prefill.hpp"
#include "planner.hpp"
#include <atomic>
#include <cstring>
#include <thread>
#include <vector>

extern "C" {
// iq, ik: int32 [n]; sq, sk: [n,r]; v: [n,dv]; out: [n,dv]; logden: [n] natural log of 1+sum W.
int dism_ref_forward_f32(const int *iq, const int *ik, int n, double tau, const float *sq,
                         const float *sk, const float *v, int r, int dv, float *out,
                         double *logden) {
    try {
        dism_prefill::Builder builder;
        builder.build(iq, ik, nullptr, size_t(n), tau);
        auto program = builder.finish();
        dism_prefill::execute<float>(program, sq, sk, v, r, dv, out);
        if (logden) std::memcpy(logden, program.logden.data(), sizeof(double) * n);
        return 0;
    } catch (...) { return 1; }
}
// `heads` independent (batch, head) sequences, each laid out as above and stored one after the other, worked off by
// `threads` host threads that take sequences from a shared counter (the pattern of the reference's own planning
// workers, planning_workers.hpp:14-85).  tau: one value per sequence.  Returns the number of rejected sequences.
int dism_ref_forward_f32_many(const int *iq, const int *ik, int heads, int n, const double *tau, const float *sq,
                              const float *sk, const float *v, int r, int dv, float *out, int threads) {
    std::atomic<int> next{0}, failed{0};
    auto work = [&] {
        for (int head = next.fetch_add(1); head < heads; head = next.fetch_add(1)) {
            const size_t at = size_t(head) * n;
            failed += dism_ref_forward_f32(iq + at, ik + at, n, tau[head], sq + at * r, sk + at * r, v + at * dv, r, dv,
                                           out + at * dv, nullptr);
        }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < threads; ++t) pool.emplace_back(work);
    work();
    for (auto &t : pool) t.join();
    return failed.load();
}
int dism_ref_forward_f64(const int *iq, const int *ik, int n, double tau, const double *sq,
                         const double *sk, const double *v, int r, int dv, double *out,
                         double *logden) {
    try {
        dism_prefill::Builder builder;
        builder.build(iq, ik, nullptr, size_t(n), tau);
        auto program = builder.finish();
        dism_prefill::execute<double>(program, sq, sk, v, r, dv, out);
        if (logden) std::memcpy(logden, program.logden.data(), sizeof(double) * n);
        return 0;
    } catch (...) { return 1; }
}
// max_j<=i L(i,j) of one sequence as the reference's decode planner tracks it: Planner::append keeps
// max_length = max(suffix-automaton match over the snapshot, diagonal band over the tail); the automaton is rebuilt
// every `interval` positions, as the planner's caller must.  keys, queries: int32 [n]; longest: int32 [n].
int dism_ref_longest_lengths(const int *keys, const int *queries, int n, int interval, int *longest) {
    try {
        dism_decode::Planner planner(1, interval, 1, 2, 0.);
        for (int p = 0; p < n; ++p) {
            if (planner.needs_rebuild()) planner.rebuild();
            planner.append(keys[p], queries[p], false);
            longest[p] = planner.max_length;
        }
        return 0;
    } catch (...) { return 1; }
}
}
