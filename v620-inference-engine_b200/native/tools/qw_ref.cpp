// qw_ref: greedy generation with the CPU fp32 reference, printing the tokens and writing one line per position
// "<pos> <next token> <logprob of next> <top-1 token> <top-1 logprob>" (the file format of the reference's
// tools/qw_ref.cpp:81-90), optionally the raw logits of the last position.
//
//   qw_ref --model DIR [--ple DIR] --prompt 1,2,3 [--new N] [--logprobs FILE] [--dump-logits FILE] [--threads N]
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../src/ref_model.hpp"

using namespace qwh;

static std::vector<float> log_softmax(const std::vector<float> &l) {
    float mx = l[0];
    for (float v : l) mx = std::max(mx, v);
    double s = 0;
    for (float v : l) s += std::exp(double(v - mx));
    const float lse = mx + float(std::log(s));
    std::vector<float> o(l.size());
    for (size_t i = 0; i < l.size(); ++i) o[i] = l[i] - lse;
    return o;
}

int main(int argc, char **argv) {
    std::string model, ple, prompt, lp_path, dump;
    int n_new = 0, threads = 0;
    for (int i = 1; i < argc; ++i) {
        auto next = [&]() -> std::string { if (i + 1 >= argc) { fprintf(stderr, "missing value for %s\n", argv[i]); exit(2); } return argv[++i]; };
        if (!strcmp(argv[i], "--model")) model = next();
        else if (!strcmp(argv[i], "--ple")) ple = next();
        else if (!strcmp(argv[i], "--prompt")) prompt = next();
        else if (!strcmp(argv[i], "--new")) n_new = atoi(next().c_str());
        else if (!strcmp(argv[i], "--logprobs")) lp_path = next();
        else if (!strcmp(argv[i], "--dump-logits")) dump = next();
        else if (!strcmp(argv[i], "--threads")) threads = atoi(next().c_str());
        else { fprintf(stderr, "unknown argument %s\n", argv[i]); return 2; }
    }
    if (model.empty() || prompt.empty()) {
        fprintf(stderr, "usage: qw_ref --model DIR [--ple DIR] --prompt 1,2,3 [--new N] [--logprobs FILE] [--dump-logits FILE]\n");
        return 2;
    }
    try {
        std::vector<int> toks;
        for (size_t p = 0; p < prompt.size();) {
            size_t q = prompt.find(',', p);
            if (q == std::string::npos) q = prompt.size();
            toks.push_back(atoi(prompt.substr(p, q - p).c_str()));
            p = q + 1;
        }
        RefModel m(model, ple, threads);
        FILE *lp = lp_path.empty() ? nullptr : fopen(lp_path.c_str(), "w");
        std::vector<float> logits;
        const int total = int(toks.size()) + n_new;
        for (int pos = 0; pos < total; ++pos) {
            if (pos >= int(toks.size())) {          // greedy: lowest index among equal maxima
                int best = 0;
                for (size_t i = 1; i < logits.size(); ++i) if (logits[i] > logits[size_t(best)]) best = int(i);
                toks.push_back(best);
                printf("%d%s", best, pos + 1 < total ? " " : "");
            }
            logits = m.forward(toks[size_t(pos)]);
            if (lp) {
                std::vector<float> ls = log_softmax(logits);
                int top = 0;
                for (size_t i = 1; i < ls.size(); ++i) if (ls[i] > ls[size_t(top)]) top = int(i);
                const int nxt = pos + 1 < int(toks.size()) ? toks[size_t(pos) + 1] : top;
                fprintf(lp, "%d %d %.6f %d %.6f\n", pos, nxt, ls[size_t(nxt)], top, ls[size_t(top)]);
            }
        }
        if (n_new) printf("\n");
        if (lp) fclose(lp);
        if (!dump.empty()) {
            FILE *f = fopen(dump.c_str(), "wb");
            fwrite(logits.data(), 4, logits.size(), f);
            fclose(f);
        }
    } catch (const std::exception &e) {
        fprintf(stderr, "qw_ref: %s\n", e.what());
        return 1;
    }
    return 0;
}
