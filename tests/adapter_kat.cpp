// The reference's own sampler test (tests/test_kernels.cpp:348-359 of paragontasx/ferro), written against the C++
// adapter exactly as the reference writes it against its Sampler class: prints the five tokens.
#include <cstdio>
#include <vector>

#include "ferro_sampler_b200.hpp"

using ferro::Sampler;
using ferro::SamplerParams;

int main() {
    const int cases[5][2] = {{-1, 0}, {-1, 2}, {2, 0}, {0, 0}, {2, 2}};   // (repeat_last_n, penalty_from)
    try {
        for (const auto& c : cases) {
            SamplerParams p;
            p.temperature = 0.0f;
            p.repetition_penalty = 2.0f;
            p.repeat_last_n = c[0];
            p.penalty_from = c[1];
            Sampler s(p);
            std::vector<float> lg = {0.f, 9.f, 10.f, 9.5f, 6.f, 0.f};
            std::printf("%d ", s.sample(lg.data(), (int)lg.size(), std::vector<int>{1, 2, 3}));
        }
        std::printf("\n");
    } catch (const std::exception& e) {
        std::printf("error: %s\n", e.what());
        return 1;
    }
    return 0;
}
