// Two models chained on the GPU through the drop-in API: the second consumes the first's results without any copy
// between host and device memory in between, and the final values equal, bit for bit, what the same chain gives
// when every result passes through host memory (the reference's way, tensor.hpp:28-168: a tensor is a host vector).
// Usage: device_chain <model_a.json> <model_b.json>     (model b takes model a's output as its input)
#include <fdeep/fdeep.hpp>

#include <cstdint>
#include <cstdio>
#include <random>

static bool same_bits(const fdeep::tensor& a, const fdeep::tensor& b) {
    return a.shape() == b.shape() && *a.as_vector() == *b.as_vector();
}

int main(int argc, char** argv) {
    if (argc < 3) {
        std::fprintf(stderr, "usage: %s model_a.json model_b.json\n", argv[0]);
        return 2;
    }
    try {
        const fdeep::model a = fdeep::load_model(argv[1], false, fdeep::dev_null_logger);
        const fdeep::model b = fdeep::load_model(argv[2], false, fdeep::dev_null_logger);
        const fdeep::tensor_shape in_shape = a.get_dummy_input_shapes().front();
        std::mt19937 rng(7);
        std::normal_distribution<float> dist(0.0f, 1.0f);
        std::vector<fdeep::tensors> samples;
        for (int s = 0; s < 5; ++s) {
            fdeep::float_vec v(in_shape.volume());
            for (float& x : v) x = dist(rng);
            samples.push_back({fdeep::tensor(in_shape, std::move(v))});
        }
        // the reference's way: every result on the host
        const fdeep::tensors host_mid = a.predict(samples[0]);
        const fdeep::tensors host_out = b.predict(host_mid);
        std::vector<fdeep::tensors> host_multi;
        for (const auto& m : a.predict_multi(samples, false)) host_multi.push_back(b.predict(m));
        if (host_mid.front().on_device()) return 10;   // nothing asked for the device: plain host tensors

        // on the device: a's results stay there, b reads them there
        a.keep_results_on_device();
        b.keep_results_on_device();
        const fdeep::tensors dev_mid = a.predict(samples[0]);
        if (!dev_mid.front().on_device()) return 11;
        std::uint64_t h2d0 = 0, d2h0 = 0, h2d1 = 0, d2h1 = 0;
        fdk_transfer_bytes(&h2d0, &d2h0);
        const fdeep::tensors dev_out = b.predict(dev_mid);
        const std::vector<fdeep::tensors> dev_multi_mid = a.predict_multi(std::vector<fdeep::tensors>{{a.to_device(samples[1][0])}}, false);
        fdk_transfer_bytes(&h2d1, &d2h1);
        // b.predict moved nothing; the to_device upload of one sample is the only host-to-device traffic in between
        if (d2h1 != d2h0) return 12;
        if (h2d1 - h2d0 != in_shape.volume() * sizeof(float)) return 13;
        if (!dev_out.front().on_device()) return 14;
        if (!same_bits(dev_out.front(), host_out.front())) return 15;       // first host access fetches the values
        if (!same_bits(dev_mid.front(), host_mid.front())) return 16;
        // several samples: one block per output shared by the results; a chained predict_multi
        const std::vector<fdeep::tensors> dev_multi = b.predict_multi(a.predict_multi(samples, true), true);
        if (dev_multi.size() != samples.size()) return 17;
        for (std::size_t s = 0; s < samples.size(); ++s)
            if (!same_bits(dev_multi[s].front(), host_multi[s].front())) return 18;
        // writing to a device-resident tensor makes its host values the current ones
        fdeep::tensor edited = a.predict(samples[2]).front();
        fdeep::tensor copy = edited;   // shares storage, as in the reference
        const fdeep::tensor_pos origin = fdeep::internal::create_tensor_shape_from_dims(std::vector<std::size_t>(edited.rank(), 1)).rank() == 1
                                             ? fdeep::tensor_pos(0) : fdeep::tensor_pos(0, 0);
        edited.set_ignore_rank(fdeep::tensor_pos(0, 0, 0, 0, 0), 42.0f);
        (void)origin;
        if (edited.on_device() || copy.on_device()) return 19;
        if (copy.get_ignore_rank(fdeep::tensor_pos(0, 0, 0, 0, 0)) != 42.0f) return 20;
        const fdeep::tensors after_edit = b.predict({edited});               // goes up from the host again
        fdeep::tensor host_edited = host_multi.empty() ? edited : a.predict(samples[2]).front();
        host_edited.set_ignore_rank(fdeep::tensor_pos(0, 0, 0, 0, 0), 42.0f);
        b.keep_results_on_device(false);
        if (!same_bits(after_edit.front(), b.predict({fdeep::tensor(host_edited.shape(), host_edited.to_vector())}).front())) return 21;
        std::printf("device chain ok: %zu values per result, no copies between the two models\n", dev_out.front().shape().volume());
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
