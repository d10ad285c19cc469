// Test driver for the C++ host (oneiron-luminal_b200/host/b200_runtime.hpp): the same calls the Python host makes, made from C++.
//
//   drive abi  <graph blob> <out.safetensors>      no GPU: header-only host compiles and links; host-only entries work
//   drive decode <desc bytes> <seed> <n new> <prompt ids...>    on a GPU: prints the greedy tokens, one line
//   drive serve <desc bytes> <seed> <len:max_new>...             on a GPU: the continuous-batching loop, one line of tokens per request
//   drive graph  <graph blob> <n>                  on a GPU: runs a primitive graph with Input 0 = 0..n-1, prints Output 2
//
// <desc bytes> is a file holding the bytes of a lum_model_desc as the Python mirror lays it out: decoding the same tokens
// from it also shows that the two hosts agree on the struct.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iterator>

#include "../../oneiron-luminal_b200/host/b200_runtime.hpp"
#include "../../oneiron-luminal_b200/host/serving.hpp"

static std::vector<uint8_t> slurp(const char* path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) { fprintf(stderr, "cannot read %s\n", path); exit(2); }
    return std::vector<uint8_t>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    const std::string mode = argv[1];
    try {
        if (mode == "abi" && argc >= 4) {
            lum_config cfg;
            lum_config_default(&cfg);
            printf("config use_graph=%d use_pdl=%d\n", cfg.use_graph, cfg.use_pdl);
            const std::vector<uint8_t> blob = slurp(argv[2]);
            lum_model_desc d;
            int64_t tok = -1, pos = -1, out = -1;
            char err[256] = {0};
            const int rc = lum_llir_describe(blob.data(), blob.size(), &d, &tok, &pos, &out, err, sizeof err);
            printf("describe rc=%d layers=%d hidden=%d vocab=%d token_input=%lld logits_output=%lld\n", rc, d.n_layers, d.hidden, d.vocab,
                   (long long)tok, (long long)out);
            // the container, host side
            const float v[6] = {1, 2, 3, 4, 5, 6};
            const char* names[1] = {"w"};
            const uint32_t dts[1] = {LUM_F32};
            const int32_t nd[1] = {2};
            const int64_t shp[8] = {2, 3};
            const void* datas[1] = {v};
            const char* mk[1] = {"made_by"};
            const char* mv[1] = {"drive.cpp"};
            if (lum_st_write(argv[3], 1, names, dts, nd, shp, datas, 1, mk, mv)) { printf("write failed: %s\n", lum_st_last_error()); return 1; }
            lum_st* st = nullptr;
            if (lum_st_open(argv[3], &st)) { printf("open failed: %s\n", lum_st_last_error()); return 1; }
            const char* nm; uint32_t dt; int32_t ndim; int64_t shape[8]; const void* data; size_t bytes;
            lum_st_tensor(st, 0, &nm, &dt, &ndim, shape, &data, &bytes);
            printf("tensor %s dtype=%u shape=%lldx%lld bytes=%zu last=%g meta=%s\n", nm, dt, (long long)shape[0], (long long)shape[1], bytes,
                   ((const float*)data)[5], lum_st_metadata(st, "made_by"));
            lum_st_close(st);
            return 0;
        }
        if (mode == "decode" && argc >= 6) {
            const std::vector<uint8_t> raw = slurp(argv[2]);
            if (raw.size() != sizeof(lum_model_desc)) { fprintf(stderr, "desc file holds %zu bytes, lum_model_desc has %zu\n", raw.size(), sizeof(lum_model_desc)); return 3; }
            lum_model_desc d;
            memcpy(&d, raw.data(), sizeof d);
            const uint64_t seed = strtoull(argv[3], nullptr, 10);
            const int n_new = atoi(argv[4]);
            std::vector<int32_t> prompt;
            for (int i = 5; i < argc; i++) prompt.push_back(atoi(argv[i]));
            lum::B200Runtime rt = lum::B200Runtime::initialize(0);
            rt.load_model(d);
            rt.synth(seed);
            rt.kv_reset();
            rt.decode_reset();
            rt.set_data(prompt);
            rt.execute({{'s', prompt.size()}, {'p', 0}});
            std::vector<int32_t> toks = {rt.get_token()};
            if (n_new > 1) {
                rt.decode_greedy(n_new - 1);
                const std::vector<int32_t> more = rt.get_decoded((size_t)n_new - 1);
                toks.insert(toks.end(), more.begin(), more.end());
            }
            printf("tokens");
            for (int32_t t : toks) printf(" %d", t);
            printf("\n");
            const std::vector<float> logits = rt.get_f32();
            printf("logits %zu launches_per_step %d\n", logits.size(), rt.stats().launches_per_step);
            // errors surface as exceptions and leave the runtime usable
            try { rt.set_dim('q', 1); printf("no exception\n"); } catch (const lum::Error& e) { printf("caught %d\n", e.code); }
            return 0;
        }
        if (mode == "serve" && argc >= 4) {
            // the C++ continuous-batching loop over the real runtime: requests "len:max_new" with seeded prompts; one line per request
            const std::vector<uint8_t> raw = slurp(argv[2]);
            if (raw.size() != sizeof(lum_model_desc)) { fprintf(stderr, "desc file holds %zu bytes, lum_model_desc has %zu\n", raw.size(), sizeof(lum_model_desc)); return 3; }
            lum_model_desc d;
            memcpy(&d, raw.data(), sizeof d);
            const uint64_t seed = strtoull(argv[3], nullptr, 10);
            lum::B200Runtime rt = lum::B200Runtime::initialize(0);
            rt.load_model(d);
            rt.synth(seed);
            lum::ContinuousBatcher<lum::B200Runtime> b(rt, 4);
            std::vector<int> ids;
            for (int i = 4; i < argc; i++) {
                int len = 0, max_new = 0;
                if (sscanf(argv[i], "%d:%d", &len, &max_new) != 2) return 2;
                std::vector<int32_t> p((size_t)len);
                for (int k = 0; k < len; k++) p[(size_t)k] = (int32_t)((11 * k + 5 * (i - 4) + 1) % d.vocab);
                ids.push_back(b.submit(p, max_new));
            }
            const auto out = b.run();
            for (int id : ids) {
                printf("request %d:", id);
                for (int32_t t : out.at(id)) printf(" %d", t);
                printf("\n");
            }
            const auto pool = rt.kv_pool();
            printf("pool %d %d %d rows_per_step %.2f\n", pool.pages_total, pool.pages_free, pool.page_rows, (double)b.rows_run / (double)b.steps_run);
            return 0;
        }
        if (mode == "graph" && argc >= 4) {
            const std::vector<uint8_t> blob = slurp(argv[2]);
            const int n = atoi(argv[3]);
            lum::B200Runtime rt = lum::B200Runtime::initialize(0);
            rt.load_llir(blob, 16, LUM_BF16);
            std::vector<float> x((size_t)n);
            for (int i = 0; i < n; i++) x[(size_t)i] = (float)i;
            rt.set_input(0, x.data(), x.size() * 4, LUM_F32);
            rt.execute({});
            const std::vector<float> y = rt.get_f32(2);
            printf("out");
            for (float v : y) printf(" %.9g", v);
            printf("\n");
            return 0;
        }
    } catch (const lum::Error& e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    fprintf(stderr, "bad arguments\n");
    return 2;
}
