// volta-b200-codegen: emits and compiles the per-model training library for the CUDA target.
//
// Stand-in for the `--target cuda` arm of Volta's `compile-train` command: where the
// reference turns an MlpTopology into a generated crate and builds one shared object per
// model (compile_mlp_train_rust_dll, src/engine/ir/codegen/mlp_train_rust_codegen.rs:143-247;
// topology checks in src/engine/executor.rs:3147-3189), this tool turns the same topology
// into a small C translation unit that exports the six volta_train_* symbols and forwards
// them to libvolta_b200, then links it with the system C compiler.
//
//   volta-b200-codegen --layers 512,1024,1024,512,256,1 --activation relu --optimizer adam
//                      [--dropout P] [--layernorm] [--clip-grad C]
//                      [--infer [--checkpoint FILE]]   (inference library exporting volta_infer, the
//                                                       checkpoint file's bytes embedded in the image)
//                      -o model.train_cuda.so [--libdir DIR] [--include DIR] [--emit-only]
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

static int index_of(const char *const *names, int n, const std::string &s) {
    for (int i = 0; i < n; ++i)
        if (s == names[i]) return i;
    return -1;
}

static std::string lower(std::string s) {
    for (auto &ch : s)
        if (ch >= 'A' && ch <= 'Z') ch = (char)(ch - 'A' + 'a');
    return s;
}

int main(int argc, char **argv) {
    std::string layers_s, act = "relu", opt = "sgd", out, libdir, incdir;
    bool emit_only = false, layernorm = false, infer = false;
    std::string ckpt;
    double dropout = 0.0, clip = 0.0;   // MlpTopology::dropout_p / use_layernorm / clip_grad
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        auto need = [&](const char *flag) -> std::string {
            if (i + 1 >= argc) { fprintf(stderr, "error: %s needs a value\n", flag); exit(2); }
            return argv[++i];
        };
        if (a == "--layers") layers_s = need("--layers");
        else if (a == "--activation") act = lower(need("--activation"));
        else if (a == "--optimizer") opt = lower(need("--optimizer"));
        else if (a == "-o") out = need("-o");
        else if (a == "--libdir") libdir = need("--libdir");
        else if (a == "--include") incdir = need("--include");
        else if (a == "--emit-only") emit_only = true;
        else if (a == "--layernorm") layernorm = true;
        else if (a == "--infer") infer = true;
        else if (a == "--checkpoint") ckpt = need("--checkpoint");
        else if (a == "--dropout") dropout = atof(need("--dropout").c_str());
        else if (a == "--clip-grad") clip = atof(need("--clip-grad").c_str());
        else { fprintf(stderr, "error: unknown argument '%s'\n", a.c_str()); return 2; }
    }
    std::vector<long> layers;
    for (size_t p = 0; p < layers_s.size();) {
        size_t q = layers_s.find(',', p);
        if (q == std::string::npos) q = layers_s.size();
        char *end = nullptr;
        long v = strtol(layers_s.substr(p, q - p).c_str(), &end, 10);
        if (v <= 0 || (end && *end)) { fprintf(stderr, "error: bad layer width in '%s'\n", layers_s.c_str()); return 2; }
        layers.push_back(v);
        p = q + 1;
    }
    // same checks, same order, as the reference's generator and executor glue
    if (layers.size() < 2) { fprintf(stderr, "error: need >= 2 layer sizes\n"); return 1; }
    if (layers.size() > 32) { fprintf(stderr, "error: at most 32 layer sizes\n"); return 1; }
    const char *acts[] = {"relu", "sigmoid", "tanh", "leaky_relu", "silu", "gelu", "softmax"};
    const char *opts[] = {"sgd", "adam", "adamw", "adagrad", "sgd_momentum"};
    if (act.empty()) act = "relu";
    if (act == "leakyrelu") act = "leaky_relu";
    int ai = index_of(acts, 7, act), oi = index_of(opts, 5, opt);
    if (ai < 0) { fprintf(stderr, "error: compile-train (cuda target) does not support activation '%s'\n", act.c_str()); return 1; }
    if (oi < 0) { fprintf(stderr, "error: compile-train (cuda target) does not support optimizer '%s'\n", opt.c_str()); return 1; }
    if (!(dropout >= 0.0 && dropout < 1.0)) { fprintf(stderr, "error: --dropout must lie in [0, 1)\n"); return 1; }
    if (!(clip >= 0.0)) { fprintf(stderr, "error: --clip-grad must not be negative\n"); return 1; }
    if (out.empty()) { fprintf(stderr, "error: -o <output library> is required\n"); return 2; }

    if (!ckpt.empty()) {
        if (!infer) { fprintf(stderr, "error: --checkpoint goes with --infer\n"); return 2; }
        FILE *c = fopen(ckpt.c_str(), "rb");
        if (!c) { fprintf(stderr, "error: cannot read checkpoint %s\n", ckpt.c_str()); return 1; }
        fclose(c);
        for (char ch : ckpt)
            if (ch == '"' || ch == '\\' || ch == '\n') { fprintf(stderr, "error: checkpoint path must not contain quotes, backslashes or newlines\n"); return 1; }
    }
    std::string src = out + ".shim.c";
    FILE *f = fopen(src.c_str(), "w");
    if (!f) { fprintf(stderr, "error: cannot write %s\n", src.c_str()); return 1; }
    if (infer) {
        // The counterpart of the reference's inference DLL (src/engine/ir/codegen/inner.rs:183-406): weights
        // embedded, one exported function.  The handle is made on the first call, for at least 64 rows, and
        // remade when a call brings more rows than it holds.
        fprintf(f, "/* generated by volta-b200-codegen --infer: layers %s, activation %s */\n", layers_s.c_str(), act.c_str());
        fprintf(f, "#include <pthread.h>\n#include <string.h>\n#include \"volta_b200.h\"\n#include \"volta_infer.h\"\n\n");
        fprintf(f, "static const int32_t k_layers[%zu] = {", layers.size());
        for (size_t i = 0; i < layers.size(); ++i) fprintf(f, "%s%ld", i ? ", " : "", layers[i]);
        fprintf(f, "};\n");
        if (!ckpt.empty()) {
            fprintf(f, "__asm__(\".section .rodata\\n.balign 16\\n.global vb_ckpt_begin\\n.hidden vb_ckpt_begin\\nvb_ckpt_begin:\\n\"\n"
                       "        \".incbin \\\"%s\\\"\\n.global vb_ckpt_end\\n.hidden vb_ckpt_end\\nvb_ckpt_end:\\n.previous\\n\");\n"
                       "extern const unsigned char vb_ckpt_begin[] __attribute__((visibility(\"hidden\")));\n"
                       "extern const unsigned char vb_ckpt_end[] __attribute__((visibility(\"hidden\")));\n", ckpt.c_str());
        }
        fprintf(f, "\nstatic vb200_handle *g_h;\nstatic int64_t g_rows;\nstatic pthread_mutex_t g_mu = PTHREAD_MUTEX_INITIALIZER;\n\n"
                   "static int ensure(int64_t rows) {\n"
                   "    vb200_config cfg;\n    vb200_handle *h = 0;\n"
                   "    if (g_h && rows <= g_rows) return 0;\n"
                   "    if (rows > 0x7fffffff) return 1;\n"
                   "    memset(&cfg, 0, sizeof cfg);\n"
                   "    cfg.n_sizes = %zu;\n    memcpy(cfg.layers, k_layers, sizeof k_layers);\n"
                   "    cfg.activation = %d;\n    cfg.use_layernorm = %d;\n    cfg.batch = rows < 64 ? 64 : (int32_t)rows;\n"
                   "    if (volta_b200_create(&cfg, &h) != 0) return 1;\n",
                layers.size(), ai, layernorm ? 1 : 0);
        if (!ckpt.empty())
            fprintf(f, "    {\n        vb200_checkpoint *ck = volta_b200_checkpoint_parse(vb_ckpt_begin, (int64_t)(vb_ckpt_end - vb_ckpt_begin));\n"
                       "        int rc = ck ? volta_b200_import_checkpoint(h, ck) : 1;\n"
                       "        volta_b200_checkpoint_free(ck);\n"
                       "        if (rc) { volta_b200_destroy(h); return 1; }\n    }\n");
        fprintf(f, "    volta_b200_destroy(g_h);\n    g_h = h;\n    g_rows = cfg.batch;\n    return 0;\n}\n\n"
                   "void volta_infer(float *input, int64_t in_n, float *output, int64_t out_n) {\n"
                   "    if (!input || !output || in_n <= 0 || in_n %% k_layers[0] != 0) return;\n"
                   "    pthread_mutex_lock(&g_mu);\n"
                   "    if (ensure(in_n / k_layers[0]) == 0) volta_b200_infer(g_h, input, in_n, output, out_n);\n"
                   "    pthread_mutex_unlock(&g_mu);\n}\n");
        fclose(f);
        f = nullptr;
    }
    if (f) {
    fprintf(f, "/* generated by volta-b200-codegen: layers %s, activation %s, optimizer %s */\n", layers_s.c_str(),
            act.c_str(), opt.c_str());
    fprintf(f, "#include <string.h>\n#include \"volta_b200.h\"\n#include \"volta_train.h\"\n\n");
    fprintf(f, "static const int32_t k_layers[%zu] = {", layers.size());
    for (size_t i = 0; i < layers.size(); ++i) fprintf(f, "%s%ld", i ? ", " : "", layers[i]);
    fprintf(f, "};\n\n");
    fprintf(f, "VoltaTrainHandle *volta_train_init(int32_t batch) {\n"
               "    vb200_config cfg;\n    vb200_handle *h = 0;\n    memset(&cfg, 0, sizeof cfg);\n"
               "    cfg.n_sizes = %zu;\n    memcpy(cfg.layers, k_layers, sizeof k_layers);\n"
               "    cfg.activation = %d;\n    cfg.optimizer = %d;\n    cfg.batch = batch;\n"
               "    cfg.use_layernorm = %d;\n    cfg.dropout_p = (float)%.9g;\n    cfg.clip_grad = (float)%.9g;\n"
               "    if (volta_b200_create(&cfg, &h) != 0) return 0;\n    return h;\n}\n\n",
            layers.size(), ai, oi, layernorm ? 1 : 0, (double)(float)dropout, (double)(float)clip);
    fprintf(f, "void volta_train_set_params(VoltaTrainHandle *h, int32_t li, const float *w, const float *b) {\n"
               "    if (h) volta_b200_set_params(h, li, w, b);\n}\n\n"
               "void volta_train_get_params(VoltaTrainHandle *h, float **wo, float **bo) {\n"
               "    if (h) volta_b200_get_params(h, wo, bo);\n}\n\n"
               "float volta_train_loss(VoltaTrainHandle *h) { return volta_b200_loss(h); }\n\n"
               "void volta_train_step(VoltaTrainHandle *h, const float *X, const float *Y, float lr) {\n"
               "    if (h) volta_b200_step(h, X, Y, lr);\n}\n\n"
               "void volta_train_free(VoltaTrainHandle *h) { volta_b200_destroy(h); }\n");
    fclose(f);
    }
    if (emit_only) { printf("%s\n", src.c_str()); return 0; }

    const char *cc = getenv("CC");
    std::string cmd = std::string(cc && *cc ? cc : "gcc") + " -O2 -shared -fPIC";
    if (!incdir.empty()) cmd += " -I'" + incdir + "'";
    cmd += " '" + src + "' -o '" + out + "'";
    if (!libdir.empty()) cmd += " -L'" + libdir + "' -Wl,-rpath,'" + libdir + "'";
    cmd += " -lvolta_b200";
    if (infer) cmd += " -lpthread";
    int rc = system(cmd.c_str());
    if (rc != 0) { fprintf(stderr, "error: compile failed; see %s\n", src.c_str()); return 1; }
    printf("%s\n", out.c_str());
    return 0;
}
