// Greedy generation through the C++ host harness (inferrous_b200/host/qwen3_model.hpp) from an on-disk bundle.
// usage: generate <bundle dir> <max tokens> <use graph 0|1> <prompt id>...      (W8A8_HEAD=w8a8 in the environment
//        runs the head as a W8A8 projection instead of the reference's bf16 head)
// Prints one line "tokens: t0 t1 ...", one line "resident decode: 0|1" (whether one-token steps ran as the single resident
// kernel; W8A8_RESIDENT_DECODE=0 turns it off) and exits 0; any failure is a message on stderr and exit code 1.
#include <cstdio>
#include <cstdlib>

#include "../../inferrous_b200/host/qwen3_model.hpp"

int main(int argc, char **argv) {
    if (argc < 5) {
        fprintf(stderr, "usage: %s <bundle dir> <max tokens> <use graph 0|1> <prompt id>...\n", argv[0]);
        return 1;
    }
    try {
        const char *head = getenv("W8A8_HEAD");
        const bool w8a8_head = head && std::string(head) == "w8a8";
        const w8a8::Qwen3Bundle bundle = w8a8::Qwen3Bundle::load(argv[1], w8a8_head ? w8a8::HeadKind::W8A8 : w8a8::HeadKind::Bf16);
        const int max_tokens = atoi(argv[2]);
        const bool use_graph = atoi(argv[3]) != 0;
        std::vector<uint32_t> prompt;
        for (int i = 4; i < argc; ++i) prompt.push_back((uint32_t)strtoul(argv[i], nullptr, 10));
        w8a8::Qwen3Model model(bundle);
        const auto out = model.generate(prompt, max_tokens, use_graph);
        printf("tokens:");
        for (uint32_t t : out.token_ids) printf(" %u", t);
        printf("\n");
        printf("resident decode: %d\n", model.resident_decode() ? 1 : 0);
        // a second request on the same model reuses caches, graph and workspaces
        const auto again = model.generate(prompt, max_tokens, use_graph);
        if (again.token_ids != out.token_ids) {
            fprintf(stderr, "second generation differs from the first\n");
            return 1;
        }
        try {
            model.generate({}, 1, use_graph);
            fprintf(stderr, "empty prompt was accepted\n");
            return 1;
        } catch (const std::invalid_argument &) {
        }
    } catch (const std::exception &e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
