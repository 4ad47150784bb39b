// CPU test of the C++ checkpoint readers (include/tpb200_formats.hpp): parses the files named
// on the command line and prints one line per tensor -- name, dtype, shape, a checksum of its
// bytes -- for the Python test to compare with its own reading of the same files; then the
// ConvRot weight resolution and the error cases.
#include <cstdio>
#include <functional>
#include <string>

#include "tpb200_cache.hpp"
#include "tpb200_formats.hpp"

static unsigned long long checksum(const uint8_t *p, size_t n) {
    unsigned long long h = 1469598103934665603ull;  // FNV-1a
    for (size_t i = 0; i < n; i++) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}

static void dump(const std::map<std::string, tpbfmt::TensorView> &ts) {
    for (const auto &kv : ts) {
        const tpbfmt::TensorView &v = kv.second;
        std::printf("T %s %s [", v.name.c_str(), v.dtype.c_str());
        for (size_t i = 0; i < v.shape.size(); i++) std::printf(i ? ",%lld" : "%lld", (long long)v.shape[i]);
        std::printf("] %zu %llu\n", v.bytes, checksum(v.data, v.bytes));
    }
}

static std::string errorName(const std::function<void()> &f) {
    try {
        f();
    } catch (const tpbfmt::Error &e) {
        return e.name;
    }
    return "none";
}

int main(int argc, char **argv) {
    if (argc < 3) return 2;
    try {
        tpbfmt::SafeTensors st(argv[1]);
        dump(st.tensors());
        // the two weights the Python test wrote: an int8 one and an int4 one
        const tpbfmt::ConvRotWeight w8 = tpbfmt::loadConvRotWeight(st, "model.blocks.0.attn.wq.weight", 64, 512);
        const tpbfmt::ConvRotWeight w4 = tpbfmt::loadConvRotWeight(st, "model.blocks.0.mlp.up.weight", 48, 256);
        std::printf("W8 %d %zu %llu %.9g\n", w8.bits, w8.w_bytes, checksum(w8.w, w8.w_bytes), (double)w8.row_scale[5]);
        std::printf("W4 %d %zu %llu %.9g\n", w4.bits, w4.w_bytes, checksum(w4.w, w4.w_bytes), (double)w4.row_scale[5]);
        std::printf("E %s %s %s\n",
                    errorName([&] { tpbfmt::loadConvRotWeight(st, "model.blocks.0.attn.wq.weight", 64, 256); }).c_str(),
                    errorName([&] { tpbfmt::loadConvRotWeight(st, "model.blocks.9.attn.wq.weight", 64, 512); }).c_str(),
                    errorName([&] { tpbfmt::loadConvRotWeight(st, "model.norm", 1, 4); }).c_str());
        tpbfmt::Gguf g(argv[2]);
        std::printf("G %u %zu %s %lld\n", g.version, g.alignment, g.strings["general.architecture"].c_str(),
                    (long long)g.integers["qwen3.block_count"]);
        dump(g.tensors());
        // name translation: "N raw arch canonical" lines, compared with the Python reader's answers
        const char *names[][2] = {{"token_embd.weight", "qwen3"}, {"output.weight", "qwen3"}, {"output_norm.weight", "qwen3"},
                                  {"blk.17.ffn_down.weight", "qwen3"}, {"blk.0.attn_k_norm.weight", "qwen3"},
                                  {"blk.0.ssm_conv1d.weight", "qwen35"}, {"blk.2.post_attention_norm.weight", "qwen3"},
                                  {"layers.3.self_attn.q_proj.weight", "qwen3"}, {"blk.0.ffn_norm.weight", "gemma3"},
                                  {"blk.0.post_ffw_norm.weight", "gemma3"}, {"blk.3.ffn_norm.weight", "qwen3"},
                                  {"blk.1.layer_output_scale.weight", "gemma4"}, {"blk.1.layer_output_scale.weight", "gemma3"},
                                  {"blk.x.attn_q.weight", "qwen3"}, {"blk.4", "qwen3"}};
        for (auto &n : names) std::printf("N %s %s %s\n", n[0], n[1], tpbfmt::canonicalName(n[0], n[1]).c_str());
        const tpbfmt::TensorView *byhf = g.get("layers.0.q4_k.weight");
        std::printf("H %d\n", byhf != nullptr && byhf == g.get("blk.0.q4_k.weight"));
        // the budgeted weight cache with a fake device: the sequence of tests/test_formats.py
        {
            std::vector<size_t> uploads;
            tpb::WeightCache<size_t> cache([&](const void *, size_t n) { uploads.push_back(n); return n; }, [](size_t &) {}, 1000);
            static char a[400], b[400], c3[300], d[900], big[2000];
            bool ok = cache.get(a, 400) == 400 && cache.get(b, 400) == 400 && cache.bytes() == 800;
            cache.get(a, 400);                       // a becomes the most recent
            cache.get(c3, 300);                      // evicts b
            ok = ok && cache.bytes() == 700 && cache.evictions == 1 && cache.hits == 1 && cache.misses == 3;
            cache.get(b, 400);                       // evicts a
            ok = ok && cache.misses == 4 && cache.bytes() == 700 && uploads == std::vector<size_t>{400, 400, 300, 400};
            cache.get(c3, 300, true);
            bool threw = false;
            try { cache.get(d, 900); } catch (const tpb::CacheFull &) { threw = true; }
            ok = ok && threw;
            cache.unpin(c3);
            cache.get(d, 900);
            ok = ok && cache.bytes() == 900;
            threw = false;
            try { cache.get(big, 2000); } catch (const tpb::CacheFull &) { threw = true; }
            ok = ok && threw;
            cache.get(d, 500);                       // same address, another size: replaced
            ok = ok && cache.bytes() == 500 && cache.misses == 8;
            std::printf("C %d\n", ok ? 1 : 0);
        }
        for (int i = 3; i < argc; i++)
            std::printf("B %s\n", errorName([&] {
                            const std::string p = argv[i];
                            if (p.size() > 5 && p.substr(p.size() - 5) == ".gguf") tpbfmt::Gguf x(p);
                            else tpbfmt::SafeTensors x(p);
                        }).c_str());
    } catch (const std::exception &e) {
        std::printf("FAIL %s\n", e.what());
        return 1;
    }
    return 0;
}
