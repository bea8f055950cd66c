// Tile selection for the B200 kernels (see autotuner.cuh).
#include "autotuner.cuh"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <tuple>

#include "common.cuh"

namespace yb {
namespace {

std::mutex g_mu;
std::map<std::tuple<uint32_t, uint32_t, uint32_t, int>, Candidate> g_cache;
TuningMode g_mode = TuningMode::Cached;
std::string g_profile_path = ".ysu_hw_profile";

std::string alnum_only(const std::string& s) {
    std::string out;
    for (char ch : s)
        if ((ch >= '0' && ch <= '9') || (ch >= 'a' && ch <= 'z') || (ch >= 'A' && ch <= 'Z')) out.push_back(ch);
    return out.empty() ? std::string("UnknownGPU") : out;
}

std::string trim(const std::string& s) {
    size_t b = s.find_first_not_of(" \t\r\n"), e = s.find_last_not_of(" \t\r\n");
    return b == std::string::npos ? std::string() : s.substr(b, e - b + 1);
}

bool parse_u32(const std::string& s, uint32_t* out) {
    std::string t = trim(s);
    if (t.empty() || t.size() > 10) return false;
    uint64_t v = 0;
    for (char ch : t) {
        if (ch < '0' || ch > '9') return false;
        v = v * 10 + (uint64_t)(ch - '0');
    }
    if (v > 0xffffffffull) return false;
    *out = (uint32_t)v;
    return true;
}

std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out;
    std::string cur;
    for (char ch : s) {
        if (ch == sep) { out.push_back(cur); cur.clear(); }
        else cur.push_back(ch);
    }
    out.push_back(cur);
    return out;
}

bool read_lines(std::vector<std::string>* lines) {
    std::ifstream f(g_profile_path);
    if (!f.good()) return false;
    std::string line;
    while (std::getline(f, line)) lines->push_back(line);
    return true;
}

}  // namespace

const char* precision_tag(Precision p) {
    switch (p) {
        case Precision::F16: return "F16";
        case Precision::F32: return "F32";
        case Precision::BF16: return "BF16";
        case Precision::Fp8: return "FP8";
        case Precision::Int4: return "INT4";
    }
    return "F16";
}

void set_tuning_mode(TuningMode m) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_mode = m;
}

// Y_AUTOTUNE = off|analytic, cached, measure|on, force|remeasure
// (src/autotuner.rs:170-186).
TuningMode tuning_mode() {
    const char* e = getenv("Y_AUTOTUNE");
    if (e) {
        std::string v(e);
        if (v == "off" || v == "analytic") return TuningMode::Analytic;
        if (v == "cached") return TuningMode::Cached;
        if (v == "measure" || v == "on") return TuningMode::Measure;
        if (v == "force" || v == "remeasure") return TuningMode::Remeasure;
        fprintf(stderr, "[Y autotuner] ignoring unknown Y_AUTOTUNE='%s' (want off|cached|measure|force)\n", e);
    }
    std::lock_guard<std::mutex> lock(g_mu);
    return g_mode;
}

void set_profile_path(const std::string& path) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_profile_path = path.empty() ? std::string(".ysu_hw_profile") : path;
}

void clear_autotune_cache() {
    std::lock_guard<std::mutex> lock(g_mu);
    g_cache.clear();
}

// Blackwell tile table. FP8 (and the 16-bit namespaces, which share the
// tcgen05 main loop shape): cta_m is the 128-lane TMEM height; cta_n is the
// UMMA N of one accumulator buffer; cta_k is one 128-byte swizzle span
// (128 e4m3 or 64 16-bit elements); stages is what fits the 227 KB of shared
// memory. INT4 decode: cta_m = tokens padded to the 8-wide MMA operand,
// cta_n = 16-column weight tile, cta_k = K covered by one ring slot
// (16 groups x 128), stages = ring slots.
std::vector<Candidate> generate_candidates(uint32_t m, uint32_t n, uint32_t k, Precision p) {
    (void)n; (void)k;
    std::vector<Candidate> out;
    if (p == Precision::Int4) {
        const uint32_t cta_m = m <= 8 ? 8 : (m <= 16 ? 16 : 32);
        if (cta_m == 32) out.push_back({32, 16, 1024, 8, 1, 6, 8});
        else out.push_back({cta_m, 16, 2048, 16, 1, cta_m == 8 ? 3u : 4u, 16});
        return out;
    }
    const uint32_t cta_k = p == Precision::Fp8 ? 128u : 64u;
    // cta_m = 256: a pair of CTAs (cluster of 2) shares each 256 x 256 tile; per CTA a
    // stage is 16 KB of A + 16 KB of B, so 6 stages fit. With a single 128-row block of A
    // the second CTA of the pair would only multiply padding.
    if (p == Precision::Fp8 && m > 128) out.push_back({256, 256, cta_k, 4, 1, 6, 4});
    out.push_back({128, 256, cta_k, 4, 1, 4, 4});
    out.push_back({128, 128, cta_k, 4, 1, 6, 4});
    out.push_back({128, 64, cta_k, 4, 1, 8, 4});
    return out;
}

bool is_launchable(const Candidate& c, uint32_t k, Precision p) {
    if (c.warps_m == 0 || c.warps_n == 0 || c.cta_k == 0) return false;
    if (p == Precision::Int4)
        return c.cta_n == 16 && (c.cta_m == 8 || c.cta_m == 16 || c.cta_m == 32) && k % 128 == 0;
    const uint32_t ebytes = p == Precision::Fp8 ? 1u : 2u;
    const bool one_cta = c.cta_m == 128 && (c.cta_n == 64 || c.cta_n == 128 || c.cta_n == 256);
    const bool cta_pair = p == Precision::Fp8 && c.cta_m == 256 && c.cta_n == 256;
    return (one_cta || cta_pair) && c.cta_k * ebytes == 128 && (k * ebytes) % 16 == 0 && c.num_stages >= 2;
}

// Analytic fallback: wave efficiency on `sm_count` persistent CTAs times the
// operand-traffic advantage of a wider tile (bytes staged per MAC fall as
// 1/cta_m + 1/cta_n). A ranking, not a measurement.
double score_candidate(const Candidate& c, uint32_t m, uint32_t n, uint32_t k, Precision p,
                       int sm_count) {
    (void)k;
    if (p == Precision::Int4) return 1.0;
    const double tiles = ceil((double)m / c.cta_m) * ceil((double)n / c.cta_n);
    const double slots = floor((double)sm_count * 128.0 / c.cta_m);  // a 256-row tile occupies two SMs
    const double waves = ceil(tiles / slots);
    const double wave_eff = tiles / (waves * slots);
    const double useful = ((double)m * n) / (tiles * c.cta_m * c.cta_n);  // ragged-edge waste
    const double traffic = 1.0 / c.cta_m + 1.0 / c.cta_n;
    return wave_eff * useful / traffic;
}

std::string persist_key(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu) {
    char buf[256];
    snprintf(buf, sizeof buf, "AUTOTUNE_%s_%ux%ux%u_%s", precision_tag(p), m, n, k,
             alnum_only(gpu).c_str());
    return buf;
}

bool parse_persisted_value(const std::string& value, Candidate* out) {
    std::vector<uint32_t> parts;
    for (const std::string& f : split(value, ',')) {
        uint32_t v;
        if (parse_u32(f, &v)) parts.push_back(v);
    }
    if (parts.size() != 6) return false;
    *out = {parts[0], parts[1], parts[2], parts[3], parts[4], parts[5], parts[3] * parts[4]};
    return true;
}

bool load_persisted(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu,
                    Candidate* out) {
    const std::string key = persist_key(m, n, k, p, gpu);
    std::vector<std::string> lines;
    if (!read_lines(&lines)) return false;
    for (const std::string& line : lines) {
        size_t eq = line.find('=');
        if (eq == std::string::npos) continue;
        if (trim(line.substr(0, eq)) == key) return parse_persisted_value(line.substr(eq + 1), out);
    }
    return false;
}

// Nearest measured shape: every dimension within 2x, closest in its worst
// dimension, and launchable at the requested K (src/autotuner.rs:293-352).
bool load_persisted_nearest(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu,
                            Candidate* out, uint32_t shape_out[3]) {
    const std::string prefix = std::string("AUTOTUNE_") + precision_tag(p) + "_";
    const std::string suffix = "_" + alnum_only(gpu);
    std::vector<std::string> lines;
    if (!read_lines(&lines)) return false;
    bool found = false;
    double best = 0.0;
    for (const std::string& line : lines) {
        size_t eq = line.find('=');
        if (eq == std::string::npos) continue;
        const std::string name = trim(line.substr(0, eq));
        if (name.size() <= prefix.size() + suffix.size()) continue;
        if (name.compare(0, prefix.size(), prefix) != 0) continue;
        if (name.compare(name.size() - suffix.size(), suffix.size(), suffix) != 0) continue;
        const std::string shape = name.substr(prefix.size(), name.size() - prefix.size() - suffix.size());
        std::vector<std::string> dims = split(shape, 'x');
        uint32_t d[3];
        if (dims.size() != 3 || !parse_u32(dims[0], &d[0]) || !parse_u32(dims[1], &d[1]) ||
            !parse_u32(dims[2], &d[2]))
            continue;
        if (d[0] == 0 || d[1] == 0 || d[2] == 0) continue;
        auto ratio = [](uint32_t a, uint32_t b) { return fabs(log((double)a / (double)b)); };
        const double dist = std::max(ratio(d[0], m), std::max(ratio(d[1], n), ratio(d[2], k)));
        if (dist > log(2.0) + 1e-12) continue;
        Candidate c;
        if (!parse_persisted_value(line.substr(eq + 1), &c)) continue;
        if (!is_launchable(c, k, p)) continue;
        if (!found || dist < best) {
            found = true;
            best = dist;
            *out = c;
            if (shape_out) { shape_out[0] = d[0]; shape_out[1] = d[1]; shape_out[2] = d[2]; }
        }
    }
    return found;
}

// Replace-or-append the KEY=VALUE line, write to a sibling temp file, rename
// over the profile (src/autotuner.rs:371-427). Unlike the reference, a missing
// profile is created: this library has no hardware-probe file to protect.
bool store_persisted(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu,
                     const Candidate& c) {
    const std::string key = persist_key(m, n, k, p, gpu);
    char val[128];
    snprintf(val, sizeof val, "%u,%u,%u,%u,%u,%u", c.cta_m, c.cta_n, c.cta_k, c.warps_m, c.warps_n,
             c.num_stages);
    const std::string entry = key + "=" + val;
    std::vector<std::string> lines;
    read_lines(&lines);
    bool replaced = false;
    for (std::string& line : lines) {
        size_t eq = line.find('=');
        if (eq != std::string::npos && trim(line.substr(0, eq)) == key) {
            line = entry;
            replaced = true;
        }
    }
    if (!replaced) lines.push_back(entry);
    const std::string tmp = g_profile_path + ".tmp";
    {
        std::ofstream f(tmp, std::ios::trunc);
        if (!f.good()) return false;
        for (const std::string& line : lines) f << line << "\n";
        f.flush();
        if (!f.good()) { remove(tmp.c_str()); return false; }
    }
    if (rename(tmp.c_str(), g_profile_path.c_str()) != 0) {
        remove(tmp.c_str());
        return false;
    }
    return true;
}

// Resolution order (src/autotuner.rs:807-990): Y_CTA_OVERRIDE, in-process
// cache, persisted exact hit, fresh measurement (if the mode allows),
// persisted nearest shape, analytic score.
Candidate autotune(uint32_t m, uint32_t n, uint32_t k, Precision p, const std::string& gpu_name,
                   int sm_count) {
    if (const char* spec = getenv("Y_CTA_OVERRIDE")) {
        Candidate c;
        if (parse_persisted_value(spec, &c)) return c;
        fprintf(stderr,
                "[Y autotuner] ignoring malformed Y_CTA_OVERRIDE='%s' "
                "(want cta_m,cta_n,cta_k,warps_m,warps_n,num_stages)\n",
                spec);
    }
    const auto key = std::make_tuple(m, n, k, (int)p);
    {
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = g_cache.find(key);
        if (it != g_cache.end()) return it->second;
    }
    auto remember = [&](const Candidate& c) {
        std::lock_guard<std::mutex> lock(g_mu);
        g_cache[key] = c;
        return c;
    };
    const TuningMode mode = tuning_mode();
    const bool may_cache = mode == TuningMode::Cached || mode == TuningMode::Measure;
    const bool may_measure = mode == TuningMode::Measure || mode == TuningMode::Remeasure;
    Candidate c;
    if (may_cache && load_persisted(m, n, k, p, gpu_name, &c) && is_launchable(c, k, p)) return remember(c);
    if (may_measure && p == Precision::Fp8) {
        std::vector<Measured> ranked;
        std::string err;
        if (tune_gemm_fp8(m, n, k, &ranked, &err) == 0 && !ranked.empty()) {
            store_persisted(m, n, k, p, gpu_name, ranked[0].candidate);
            return remember(ranked[0].candidate);
        }
        fprintf(stderr, "[Y autotuner] could not measure M=%u N=%u K=%u (%s); using the analytic score\n",
                m, n, k, err.c_str());
    }
    if (may_cache && load_persisted_nearest(m, n, k, p, gpu_name, &c, nullptr)) return remember(c);
    std::vector<Candidate> cands = generate_candidates(m, n, k, p);
    Candidate best = cands[0];
    double best_score = -1.0;
    for (const Candidate& cand : cands) {
        if (!is_launchable(cand, k, p)) continue;
        const double s = score_candidate(cand, m, n, k, p, sm_count);
        if (s > best_score) { best_score = s; best = cand; }
    }
    return remember(best);
}

// ---- measurement discipline ---------------------------------------------------
// Two candidates are separable only if their fastest rounds differ by more
// than this run's own dispersion (median - best), floored at 0.25% of the
// time (src/empirical_autotune.rs:153-188).
bool Timing::tied_with(const Timing& o) const {
    double noise = std::max(median_us - best_us, o.median_us - o.best_us);
    noise = std::max(noise, 0.0025 * std::min(best_us, o.best_us));
    return fabs(best_us - o.best_us) <= noise;
}

double median(std::vector<double> v) {
    if (v.empty()) return INFINITY;
    std::sort(v.begin(), v.end());
    const size_t n = v.size();
    return n % 2 ? v[n / 2] : (v[n / 2 - 1] + v[n / 2]) / 2.0;
}

// `results` is sorted fastest first. Among candidates tied with the fastest,
// prefer the warp count closest to four, then the deeper K tile, then the
// measured time, then the larger tile (src/empirical_autotune.rs:922-949).
size_t select_winner(const std::vector<Measured>& results) {
    if (results.empty()) return 0;
    const Timing best = results[0].timing;
    auto key = [](const Measured& r) {
        return std::make_tuple(-llabs((long long)r.candidate.num_warps - 4), r.candidate.cta_k,
                               -(long long)(r.timing.best_us * 1000.0), r.candidate.cta_m,
                               r.candidate.cta_n);
    };
    size_t winner = 0;
    for (size_t i = 1; i < results.size(); ++i) {
        if (!results[i].timing.tied_with(best)) continue;
        if (key(results[i]) > key(results[winner])) winner = i;
    }
    return winner;
}

// How many distinct copies of the streamed operand to rotate over so a timing
// loop measures HBM, not L2: enough to reach 4x L2, capped by the replica
// limit and by 60% of free memory (src/empirical_autotune.rs:398-440). The cap
// is 64 rather than the reference's 8: B200's 126 MB L2 is several times a
// 23 MB INT4 weight matrix.
size_t plan_weight_replicas(size_t b_bytes, size_t a_bytes, size_t c_bytes, size_t l2_bytes,
                            size_t free_bytes) {
    constexpr size_t kOversubscribe = 4, kMaxReplicas = 64;
    if (b_bytes == 0 || l2_bytes == 0) return 1;
    const size_t target = l2_bytes * kOversubscribe;
    if (a_bytes + b_bytes >= target) return 1;
    size_t wanted = (target - a_bytes + b_bytes - 1) / b_bytes;
    wanted = std::max<size_t>(1, std::min(wanted, kMaxReplicas));
    const size_t budget = (size_t)((double)free_bytes * 0.6);
    const size_t fixed = a_bytes + c_bytes;
    if (budget <= fixed + b_bytes) return 1;
    const size_t affordable = (budget - fixed) / b_bytes;
    return std::min(wanted, std::max<size_t>(affordable, 1));
}

std::string current_gpu_name() {
    static std::mutex mu;
    static std::map<int, std::string> names;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return "NVIDIA B200";
    }
    std::lock_guard<std::mutex> lock(mu);
    auto it = names.find(dev);
    if (it != names.end()) return it->second;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return "NVIDIA B200";
    }
    names[dev] = prop.name;
    return names[dev];
}

// ---- on-device tuning of the FP8 GEMM -------------------------------------------
namespace {

float e4m3_to_float(uint8_t code) {
    const int sign = code >> 7, exp = (code >> 3) & 0xf, mant = code & 7;
    float v;
    if (exp == 0xf && mant == 7) return NAN;
    if (exp == 0) v = (float)mant / 512.0f;
    else v = ldexpf((float)(8 + mant), exp - 10);
    return sign ? -v : v;
}

struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
    int alloc(size_t bytes) { return check_cuda(cudaMalloc(&p, bytes), "cudaMalloc"); }
};

}  // namespace

int tune_gemm_fp8(uint32_t m, uint32_t n, uint32_t k, std::vector<Measured>* out, std::string* error) {
    auto bail = [&](const char* what) {
        if (error) *error = std::string(what) + ": " + y_b200_last_error();
        return -1;
    };
    out->clear();
    const size_t a_elems = (size_t)m * k, b_elems = (size_t)n * k;
    DevBuf a16, b16, aq, bq, c, scale;
    if (a16.alloc(a_elems * 2) || b16.alloc(b_elems * 2) || aq.alloc(a_elems) || bq.alloc(b_elems) ||
        c.alloc((size_t)m * n * 2) || scale.alloc(256))
        return bail("allocation");
    // Inputs: the reference's generator (|v| in [1/8, 1)), quantised with
    // scale 1/256 so every code is a normal e4m3 value.
    const float s = 1.0f / 256.0f;
    if (y_b200_fill_random_f16(a16.p, a_elems, 0, 0xA5A5123456789ABCull, nullptr) ||
        y_b200_fill_random_f16(b16.p, b_elems, 0, 0xB1B10FEDCBA98765ull, nullptr))
        return bail("fill");
    if (check_cuda(cudaMemcpy(scale.p, &s, 4, cudaMemcpyHostToDevice), "cudaMemcpy")) return bail("scale");
    if (y_b200_quantize_fp8(a16.p, Y_B200_F16, a_elems, (const float*)scale.p, aq.p, nullptr) ||
        y_b200_quantize_fp8(b16.p, Y_B200_F16, b_elems, (const float*)scale.p, bq.p, nullptr))
        return bail("quantise");

    // 48 sampled outputs checked against f64 dot products (rel-L2 < 2e-2).
    constexpr int kSamples = 48;
    std::vector<uint8_t> arow(k), brow(k);
    std::vector<std::pair<uint32_t, uint32_t>> pos;
    std::vector<double> ref;
    for (int i = 0; i < kSamples; ++i) {
        uint64_t z = (uint64_t)(i + 1) * 0x9E3779B97F4A7C15ull;
        z ^= z >> 29;
        const uint32_t r = (uint32_t)(z % m), col = (uint32_t)((z >> 32) % n);
        if (check_cuda(cudaMemcpy(arow.data(), (uint8_t*)aq.p + (size_t)r * k, k, cudaMemcpyDeviceToHost), "cudaMemcpy") ||
            check_cuda(cudaMemcpy(brow.data(), (uint8_t*)bq.p + (size_t)col * k, k, cudaMemcpyDeviceToHost), "cudaMemcpy"))
            return bail("sample download");
        double acc = 0.0;
        for (uint32_t kk = 0; kk < k; ++kk) acc += (double)e4m3_to_float(arow[kk]) * (double)e4m3_to_float(brow[kk]);
        pos.push_back({r, col});
        ref.push_back(acc * (double)s * (double)s);
    }

    struct Live { Candidate cand; y_b200_gemm_fp8_args args; };
    std::vector<Live> live;
    for (const Candidate& cand : generate_candidates(m, n, k, Precision::Fp8)) {
        if (!is_launchable(cand, k, Precision::Fp8)) continue;
        y_b200_gemm_fp8_args g = {};
        g.a = aq.p; g.bt = bq.p; g.c = c.p;
        g.m = (int)m; g.n = (int)n; g.k = (int)k;
        g.scale_a = s; g.scale_b = s;
        g.out_kind = Y_B200_BF16;
        g.cta_n = (int)cand.cta_n;
        g.cta_m = (int)cand.cta_m;
        if (y_b200_gemm_fp8(&g, nullptr) || y_b200_device_status(nullptr)) continue;
        double num = 0.0, den = 0.0;
        bool ok = true;
        for (int i = 0; i < kSamples && ok; ++i) {
            uint16_t bits;
            ok = cudaMemcpy(&bits, (uint16_t*)c.p + (size_t)pos[i].first * n + pos[i].second, 2,
                            cudaMemcpyDeviceToHost) == cudaSuccess;
            uint32_t u = (uint32_t)bits << 16;
            float got;
            memcpy(&got, &u, 4);
            num += ((double)got - ref[i]) * ((double)got - ref[i]);
            den += ref[i] * ref[i];
        }
        if (!ok || !(sqrt(num / std::max(den, 1e-300)) < 2e-2)) continue;
        live.push_back({cand, g});
    }
    if (live.empty()) {
        if (error) *error = "no candidate launched and verified";
        return -1;
    }

    cudaEvent_t e0, e1;
    if (check_cuda(cudaEventCreate(&e0), "cudaEventCreate") || check_cuda(cudaEventCreate(&e1), "cudaEventCreate"))
        return bail("events");
    auto time_batch = [&](const Live& l, int iters) -> double {
        cudaDeviceSynchronize();
        cudaEventRecord(e0, nullptr);
        for (int i = 0; i < iters; ++i) y_b200_gemm_fp8(&l.args, nullptr);
        cudaEventRecord(e1, nullptr);
        cudaEventSynchronize(e1);
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        return (double)ms * 1000.0 / iters;
    };
    // Clock ramp, then interleaved rounds with a rotating start; rank by the
    // fastest round (src/empirical_autotune.rs:727-757, :836-870).
    {
        cudaEvent_t r0, r1;
        cudaEventCreate(&r0); cudaEventCreate(&r1);
        cudaEventRecord(r0, nullptr);
        float ms = 0.0f;
        int guard = 0;
        while (ms < 1000.0f && guard++ < 100000) {
            y_b200_gemm_fp8(&live[0].args, nullptr);
            if ((guard & 15) == 0) { cudaEventRecord(r1, nullptr); cudaEventSynchronize(r1); cudaEventElapsedTime(&ms, r0, r1); }
        }
        cudaEventDestroy(r0); cudaEventDestroy(r1);
    }
    constexpr int kRounds = 15;
    std::vector<int> iters;
    for (const Live& l : live) {
        const double per = time_batch(l, 3);
        iters.push_back(std::max(3, std::min(500, (int)ceil(10000.0 / std::max(per, 1e-3)))));
    }
    std::vector<std::vector<double>> samples(live.size());
    for (int round = 0; round < kRounds; ++round)
        for (size_t off = 0; off < live.size(); ++off) {
            const size_t slot = (off + (size_t)round) % live.size();
            samples[slot].push_back(time_batch(live[slot], iters[slot]));
        }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    const double flops = 2.0 * m * (double)n * k;
    for (size_t i = 0; i < live.size(); ++i) {
        Timing t;
        t.best_us = *std::min_element(samples[i].begin(), samples[i].end());
        t.max_us = *std::max_element(samples[i].begin(), samples[i].end());
        t.median_us = median(samples[i]);
        out->push_back({live[i].cand, t, flops / (t.best_us * 1e-6) / 1e12, true});
    }
    std::sort(out->begin(), out->end(),
              [](const Measured& a, const Measured& b) { return a.timing.best_us < b.timing.best_us; });
    std::swap((*out)[0], (*out)[select_winner(*out)]);
    return 0;
}

}  // namespace yb
