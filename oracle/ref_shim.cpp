// C-ABI shim around the reference's own native CPU hard forward (test infrastructure only).
//
// Compiled from the reference sources where they lie (never copied into this repository):
//   dism_v3/python/flash_dism/inference/csrc/prefill.hpp  Builder (:426-515), finish (:517-599),
//   execute<T> (:603-625).  The build recipe is oracle/Makefile; the output goes to oracle/_ref/.
// One call plans and executes one (batch, head) sequence: labels -> Program -> output rows.
#include "prefill.hpp"
#include <cstring>

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
}
