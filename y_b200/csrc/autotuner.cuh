// Tile selection for the B200 kernels: candidate table, analytic score,
// per-(shape, precision, GPU) cache persisted in the reference's
// `.ysu_hw_profile` line format, and the measured (on-device) selector.
#pragma once

#include <stdint.h>

#include <string>
#include <vector>

namespace yb {

// Cache namespaces. F16/F32/BF16/FP8 are the reference's tags
// (src/autotuner.rs:48-96); INT4 is new (weight-only decode GEMM).
enum class Precision { F16, F32, BF16, Fp8, Int4 };
const char* precision_tag(Precision p);

// Same six persisted integers as the reference's AutotuneCandidate
// (src/autotuner.rs:57-82); num_warps = warps_m * warps_n counts the warps
// that own output rows (the epilogue warps of the FP8 GEMM, the consumer warps
// of the decode GEMM); producer / MMA-issuer warps come on top.
struct Candidate {
    uint32_t cta_m, cta_n, cta_k, warps_m, warps_n, num_stages, num_warps;
    bool operator==(const Candidate& o) const {
        return cta_m == o.cta_m && cta_n == o.cta_n && cta_k == o.cta_k && warps_m == o.warps_m &&
               warps_n == o.warps_n && num_stages == o.num_stages && num_warps == o.num_warps;
    }
};

enum class TuningMode { Cached, Analytic, Measure, Remeasure };
void set_tuning_mode(TuningMode m);
TuningMode tuning_mode();  // Y_AUTOTUNE overrides the process-wide mode

std::vector<Candidate> generate_candidates(uint32_t m, uint32_t n, uint32_t k, Precision p);
bool is_launchable(const Candidate& c, uint32_t k, Precision p);
double score_candidate(const Candidate& c, uint32_t m, uint32_t n, uint32_t k, Precision p,
                       int sm_count);
Candidate autotune(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu_name,
                   int sm_count);
void clear_autotune_cache();

// Persistence (src/autotuner.rs:227-427).
void set_profile_path(const std::string& path);
std::string persist_key(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu);
bool parse_persisted_value(const std::string& value, Candidate* out);
bool load_persisted(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu,
                    Candidate* out);
bool load_persisted_nearest(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu,
                            Candidate* out, uint32_t shape_out[3]);
bool store_persisted(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu,
                     const Candidate& c);

// Measurement discipline (src/empirical_autotune.rs).
struct Timing {
    double best_us, median_us, max_us;
    bool tied_with(const Timing& o) const;
};
struct Measured {
    Candidate candidate;
    Timing timing;
    double tflops;
    bool finalist;
};
size_t select_winner(const std::vector<Measured>& results);
size_t plan_weight_replicas(size_t b_bytes, size_t a_bytes, size_t c_bytes, size_t l2_bytes,
                            size_t free_bytes);
double median(std::vector<double> v);
// On-device tuning of the FP8 GEMM at one shape: every launchable candidate is
// verified against sampled f64 dot products, then timed interleaved.
int tune_gemm_fp8(uint32_t m, uint32_t n, uint32_t k, std::vector<Measured>* out,
                  std::string* error);

std::string current_gpu_name();

}  // namespace yb
