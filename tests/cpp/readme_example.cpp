// Mirrors the reference's test/readme_example_main.cpp and test/test_model_*_test.cpp through the
// drop-in header: load a model (with its embedded self test), predict, predict_multi sequentially and
// "parallelly" on dummy inputs, and print the result.  Usage: readme_example <model.json>
#include <fdeep/fdeep.hpp>

int main(int argc, char** argv) {
    if (argc < 2) {
        std::cerr << "usage: readme_example model.json" << std::endl;
        return 2;
    }
    try {
        const auto model = fdeep::load_model(argv[1], true, fdeep::cout_logger, static_cast<fdeep::float_type>(0.0001));
        const auto result = model.predict({fdeep::tensor(fdeep::tensor_shape(static_cast<std::size_t>(4)), fdeep::float_vec{1, 2, 3, 4})});
        std::cout << fdeep::show_tensors(result) << std::endl;
        const std::size_t n = 10;
        const auto multi_inputs = std::vector<fdeep::tensors>(n, model.generate_dummy_inputs());
        const auto a = model.predict_multi(multi_inputs, false);
        const auto b = model.predict_multi(multi_inputs, true);
        if (a.size() != n || b.size() != n) return 3;
        for (std::size_t i = 0; i < n; ++i)
            if (*a[i][0].as_vector() != *b[i][0].as_vector()) return 4;
        std::cout << "class " << model.predict_class({fdeep::tensor(fdeep::tensor_shape(static_cast<std::size_t>(4)), fdeep::float_vec{1, 2, 3, 4})})
                  << " name " << model.name() << " inputs " << fdeep::show_tensor_shapes_variable(model.get_input_shapes()) << std::endl;
        std::cout << "test_speed " << model.test_speed() << " s" << std::endl;
    } catch (const std::exception& e) {
        std::cerr << "error: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
