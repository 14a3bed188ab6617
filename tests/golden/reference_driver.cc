// Runs the reference engine's own CPU forward on given token ids and writes the logits.
//
//   reference_driver <model.json> <model.bin> <normal|neox> <out.f32> <token> [<token> ...]
//
// Test infrastructure for tests/golden/make_golden.py: it is compiled against the reference's static
// library (libyan_minillama.a, CPU build) where the reference checkout is mounted, and is not part of
// the product.  The reference's command line feeds text through its tokenizers and has no switch for
// the pairing of rotary dimensions; this driver feeds arbitrary ids one token per forward, as the
// reference's prefill does (src/forward.cc:473-488), and sets `rope_type` on the loaded model the way
// the reference's own tests do (test/forward_test.cc:258-261).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "include/batch.h"
#include "include/context.h"
#include "include/forward.h"
#include "include/load.h"
#include "include/model.h"

int main(int argc, char** argv) {
    if (argc < 6) {
        std::fprintf(stderr, "usage: %s model.json model.bin normal|neox out.f32 token...\n", argv[0]);
        return 2;
    }
    yan_lamma::Model model = yan_lamma::ParseModel(argv[1], argv[2]);
    if (!model.is_loaded) {
        std::fprintf(stderr, "load failed: %s\n", model.load_error_.c_str());
        return 1;
    }
    model.config.rope_type = std::strcmp(argv[3], "neox") == 0 ? yan_lamma::RopeType::kNeoX : yan_lamma::RopeType::kNormal;
    yan_lamma::Context context(&model);
    std::FILE* out = std::fopen(argv[4], "wb");
    if (out == nullptr) return 1;
    for (int i = 5; i < argc; ++i) {
        const int token = std::atoi(argv[i]);
        const yan_lamma::Tensor logits = yan_lamma::ForwardBatch(model, context, yan_lamma::Batch::Single(token, i - 5));
        std::fwrite(logits.data.data(), sizeof(float), logits.data.size(), out);
    }
    std::fclose(out);
    return 0;
}
