// A consumer of the engine ABI written against the REFERENCE's own C++ wrapper (include/tenzo.hpp of catdlia/tenzo:
// tenzo::Engine, RAII over the C API) - compiled with the reference's include directory and linked against this
// repository's libtenzo_runtime.so, it shows the library is a drop-in at the source level: same headers, same calls,
// same loop as the reference's examples/basic_inference.cpp:143-171 (prefill all but the last prompt token, then
// generate). The model dimensions come from the command line so that a small synthetic checkpoint can be used.
//
//   hpp_consumer <weights.bin> <model.mlir> <hidden> <q_heads> <kv_heads> <layers> <ffn> <vocab> <max_seq> <n_gen> <tok>...
//
// Prints the generated token ids on one line.
#include <tenzo.hpp>

#include <cstdlib>
#include <iostream>
#include <vector>

int main(int argc, char** argv) {
    if (argc < 12) {
        std::cerr << "usage: hpp_consumer weights.bin model.mlir hidden q_heads kv_heads layers ffn vocab max_seq n_gen tok..." << std::endl;
        return 2;
    }
    tenzo_config_t config = tenzo_default_config();
    config.hidden_size = std::atoi(argv[3]);
    config.num_q_heads = std::atoi(argv[4]);
    config.num_kv_heads = std::atoi(argv[5]);
    config.num_layers = std::atoi(argv[6]);
    config.ffn_dim = std::atoi(argv[7]);
    config.vocab_size = std::atoi(argv[8]);
    config.max_seq_len = std::atoi(argv[9]);
    const int n_gen = std::atoi(argv[10]);
    std::vector<int> prompt;
    for (int i = 11; i < argc; ++i) prompt.push_back(std::atoi(argv[i]));
    try {
        tenzo::Engine engine(config);
        engine.load_model(argv[1], argv[2]);
        for (size_t i = 0; i + 1 < prompt.size(); ++i) engine.prefill_token(prompt[i]);
        tenzo_sampling_params_t params = tenzo_default_sampling_params();
        params.temperature = 0.0f;
        params.repetition_penalty = 1.0f;
        std::vector<int> all = prompt;
        int cur = prompt.back();
        for (int s = 0; s < n_gen; ++s) {
            const int next = engine.generate_step(cur, params, all);
            all.push_back(next);
            std::cout << next << (s + 1 < n_gen ? " " : "\n");
            cur = next;
        }
        if (engine.get_seq_len() != static_cast<int>(prompt.size()) - 1 + n_gen) return 3;
    } catch (const std::exception& e) {
        std::cerr << "error: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
