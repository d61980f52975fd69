// Driver for the REFERENCE itself (test infrastructure; compiled only when its dependencies are at hand).
//
// Links against nothing of this repository: it includes the reference's own <fdeep/fdeep.hpp> (Dobiasd/frugally-deep,
// header-only; needs Eigen 3.4.0, FunctionalPlus 0.2.24 and nlohmann/json on the include path), loads a converted
// model file with fdeep::load_model and runs fdeep::model::predict on the samples of an input file, writing the
// results to an output file.  oracle/build_ref.py compiles it into oracle/_ref/ and uses it to check the CPU
// restatement (oracle/fdeep_oracle.cpp) against the reference on every golden fixture, and as the timed CPU arm.
//
//   ref_driver <model.json> <inputs.bin> <outputs.bin> [repeat]
//
// File format (little endian): int64 n_samples, int64 tensors per sample, then per tensor: int64 rank, rank x int64
// dims, volume x float32.  The output file has the same format.  With `repeat` > 1 the whole batch is run through
// predict_multi that many times and the seconds per pass are printed (the timed CPU arm of the benchmark).
#include <fdeep/fdeep.hpp>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <vector>

static std::int64_t read_i64(std::ifstream& f) {
    std::int64_t v = 0;
    f.read(reinterpret_cast<char*>(&v), sizeof(v));
    return v;
}
static void write_i64(std::ofstream& f, std::int64_t v) { f.write(reinterpret_cast<const char*>(&v), sizeof(v)); }

int main(int argc, char** argv) {
    if (argc < 4) {
        std::fprintf(stderr, "usage: %s model.json inputs.bin outputs.bin [repeat]\n", argv[0]);
        return 2;
    }
    try {
        const auto model = fdeep::load_model(argv[1], true, fdeep::dev_null_logger);
        std::ifstream in(argv[2], std::ios::binary);
        if (!in.good()) throw std::runtime_error("cannot open the input file");
        const std::int64_t n_samples = read_i64(in), per_sample = read_i64(in);
        std::vector<fdeep::tensors> samples;
        for (std::int64_t s = 0; s < n_samples; ++s) {
            fdeep::tensors ts;
            for (std::int64_t i = 0; i < per_sample; ++i) {
                const std::int64_t rank = read_i64(in);
                std::vector<std::size_t> dims;
                for (std::int64_t d = 0; d < rank; ++d) dims.push_back(static_cast<std::size_t>(read_i64(in)));
                const fdeep::tensor_shape shape = fdeep::internal::create_tensor_shape_from_dims(dims);
                std::vector<float> values(shape.volume());
                in.read(reinterpret_cast<char*>(values.data()), static_cast<std::streamsize>(values.size() * sizeof(float)));
                ts.push_back(fdeep::tensor(shape, fdeep::float_vec(values.begin(), values.end())));
            }
            samples.push_back(ts);
        }
        const int repeat = argc > 4 ? std::atoi(argv[4]) : 1;
        std::vector<fdeep::tensors> results;
        const auto t0 = std::chrono::steady_clock::now();
        for (int r = 0; r < (repeat > 1 ? repeat : 1); ++r) results = model.predict_multi(samples, true);
        const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (repeat > 1) std::printf("seconds_per_pass %.6f samples %lld\n", dt / repeat, static_cast<long long>(n_samples));
        std::ofstream out(argv[3], std::ios::binary);
        write_i64(out, static_cast<std::int64_t>(results.size()));
        write_i64(out, results.empty() ? 0 : static_cast<std::int64_t>(results.front().size()));
        for (const auto& ts : results)
            for (const auto& t : ts) {
                const auto dims = t.shape().dimensions();
                write_i64(out, static_cast<std::int64_t>(dims.size()));
                for (std::size_t d : dims) write_i64(out, static_cast<std::int64_t>(d));
                const std::vector<float> values = t.to_vector();
                out.write(reinterpret_cast<const char*>(values.data()), static_cast<std::streamsize>(values.size() * sizeof(float)));
            }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
