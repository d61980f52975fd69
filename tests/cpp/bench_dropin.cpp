// End-to-end timing through the drop-in C++ API, written the way a user of the reference writes it
// (README.md:124-135 of the reference; model.hpp:31-42): fdeep::load_model, one separately allocated fdeep::tensor per
// sample (ordinary pageable std::vector storage), model.predict_multi, results read on the host.
//
//   bench_dropin <model.json> <samples> <steps> <dim> [<dim> ...]
//
// Prints one JSON object: samples per second over `steps` timed calls (after two warm-up calls), the model's load
// time, and a checksum of the last results so that the work cannot be skipped.
#include <fdeep/fdeep.hpp>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>

int main(int argc, char** argv) {
    if (argc < 5) {
        std::fprintf(stderr, "usage: %s <model.json> <samples> <steps> <dim> [<dim> ...]\n", argv[0]);
        return 2;
    }
    try {
        const std::size_t n = (std::size_t)std::atoll(argv[2]);
        const int steps = std::atoi(argv[3]);
        std::vector<std::size_t> dims;
        for (int i = 4; i < argc; ++i) dims.push_back((std::size_t)std::atoll(argv[i]));
        const fdeep::tensor_shape shape = fdeep::internal::create_tensor_shape_from_dims(dims);
        const auto t_load = std::chrono::steady_clock::now();
        const fdeep::model model = fdeep::load_model(argv[1], false, fdeep::dev_null_logger);
        const double load_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_load).count();
        std::mt19937 rng(1);
        std::normal_distribution<float> dist(0.0f, 1.0f);
        std::vector<fdeep::tensors> inputs;
        inputs.reserve(n);
        for (std::size_t s = 0; s < n; ++s) {
            fdeep::float_vec v(shape.volume());
            for (float& x : v) x = dist(rng);
            inputs.push_back({fdeep::tensor(shape, std::move(v))});
        }
        double checksum = 0.0;
        for (int warm = 0; warm < 2; ++warm) model.predict_multi(inputs, true);
        const auto t0 = std::chrono::steady_clock::now();
        for (int it = 0; it < steps; ++it) {
            const std::vector<fdeep::tensors> out = model.predict_multi(inputs, true);
            checksum = 0.0;
            for (const auto& o : out) checksum += (double)o.front().as_vector()->front();
        }
        const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        std::printf("{\"value\": %.3f, \"unit\": \"samples/s\", \"samples\": %zu, \"steps\": %d, \"model_load_s\": %.3f, \"checksum\": %.6g, "
                    "\"entry\": \"fdeep::model::predict_multi over separately allocated pageable fdeep::tensor objects\"}\n",
                    (double)n * steps / dt, n, steps, load_s, checksum);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
