// Command-line host of the C++ API: loads an `.npz` BERT archive and serves requests with no Python in the process
// (the role of example/cpp/bert_model_example.cpp in the reference, which ran one fixed request and a thread demo).
//
//   bert_model_example MODEL.npz N_LAYERS N_HEADS [--dtype float32|float16|bfloat16] [--ids FILE] [--out FILE]
//                      [--pooler] [--devices K] [--requests R] [--batch B] [--seq L] [--vocab V]
//
//   --ids FILE   one request per line, token ids separated by spaces; without it, --batch random requests of --seq tokens
//   --out FILE   the result as raw little-endian float32 ([batch, longest, hidden], or [batch, hidden] with --pooler)
//   --devices K  one model and one host thread per device 0..K-1, each running --requests batches; prints sequences/s
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "bert_model.h"
#include "core.h"

namespace {

struct Args {
  std::string model, dtype = "float32", ids_file, out_file;
  size_t n_layers = 12;
  int64_t n_heads = 12, batch = 1, seq = 128, vocab = 30522;
  int devices = 1, requests = 1;
  bool pooler = false;
};

bool Parse(int argc, char** argv, Args* a) {
  if (argc < 4) return false;
  a->model = argv[1];
  a->n_layers = (size_t)std::atoll(argv[2]);
  a->n_heads = std::atoll(argv[3]);
  for (int i = 4; i < argc; ++i) {
    const std::string k = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (k == "--dtype") a->dtype = next();
    else if (k == "--ids") a->ids_file = next();
    else if (k == "--out") a->out_file = next();
    else if (k == "--pooler") a->pooler = true;
    else if (k == "--devices") a->devices = std::atoi(next());
    else if (k == "--requests") a->requests = std::atoi(next());
    else if (k == "--batch") a->batch = std::atoll(next());
    else if (k == "--seq") a->seq = std::atoll(next());
    else if (k == "--vocab") a->vocab = std::atoll(next());
    else return false;
  }
  return a->devices >= 1 && a->requests >= 1 && a->batch >= 1 && a->seq >= 1;
}

std::vector<std::vector<int64_t>> ReadIds(const std::string& path) {
  std::ifstream f(path);
  if (!f.good()) throw std::runtime_error("cannot open " + path);
  std::vector<std::vector<int64_t>> rows;
  std::string line;
  while (std::getline(f, line)) {
    std::istringstream ss(line);
    std::vector<int64_t> row;
    int64_t v;
    while (ss >> v) row.push_back(v);
    if (!row.empty()) rows.push_back(std::move(row));
  }
  return rows;
}

std::vector<std::vector<int64_t>> RandomIds(int64_t batch, int64_t seq, int64_t vocab, uint64_t seed) {
  std::vector<std::vector<int64_t>> rows((size_t)batch, std::vector<int64_t>((size_t)seq));
  uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
  for (auto& r : rows)
    for (auto& v : r) {
      s = s * 6364136223846793005ull + 1442695040888963407ull;
      v = (int64_t)((s >> 33) % (uint64_t)vocab);
    }
  return rows;
}

}  // namespace

int main(int argc, char** argv) {
  Args a;
  if (!Parse(argc, argv, &a)) {
    std::fprintf(stderr,
                 "usage: %s MODEL.npz N_LAYERS N_HEADS [--dtype float32|float16|bfloat16] [--ids FILE] [--out FILE] [--pooler]\n"
                 "          [--devices K] [--requests R] [--batch B] [--seq L] [--vocab V]\n",
                 argv[0]);
    return 2;
  }
  try {
    const auto ids = a.ids_file.empty() ? RandomIds(a.batch, a.seq, a.vocab, 1) : ReadIds(a.ids_file);
    if (a.devices == 1 && a.requests == 1) {
      BertModel model(a.model, kDLCUDA, a.n_layers, a.n_heads, a.dtype, 0);
      const std::vector<float> out = model(ids, {}, {}, PoolType::kFirst, a.pooler);
      double sum = 0;
      for (float v : out) sum += v;
      std::printf("%zu values, sum %.6f, first %.6f %.6f %.6f\n", out.size(), sum, out.size() > 0 ? out[0] : 0.f, out.size() > 1 ? out[1] : 0.f,
                  out.size() > 2 ? out[2] : 0.f);
      if (!a.out_file.empty()) {
        std::ofstream f(a.out_file, std::ios::binary);
        f.write(reinterpret_cast<const char*>(out.data()), (std::streamsize)(out.size() * sizeof(float)));
      }
      return 0;
    }
    // serving loop: one model and one host thread per device, requests sharded by device (weights replicated, no
    // communication between devices)
    std::vector<std::unique_ptr<BertModel>> models;
    for (int d = 0; d < a.devices; ++d) models.emplace_back(new BertModel(a.model, kDLCUDA, a.n_layers, a.n_heads, a.dtype, d));
    std::vector<std::string> errors((size_t)a.devices);
    for (int pass = 0; pass < 2; ++pass) {  // pass 0 warms up
      const int reps = pass == 0 ? 2 : a.requests;
      const auto t0 = std::chrono::steady_clock::now();
      std::vector<std::thread> threads;
      for (int d = 0; d < a.devices; ++d)
        threads.emplace_back([&, d] {
          try {
            for (int r = 0; r < reps; ++r) (*models[(size_t)d])(ids, {}, {}, PoolType::kFirst, true);
          } catch (const std::exception& e) {
            errors[(size_t)d] = e.what();
          }
        });
      for (auto& t : threads) t.join();
      for (const auto& e : errors)
        if (!e.empty()) throw std::runtime_error(e);
      const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      if (pass == 1)
        std::printf("%d device(s) x %d batches of %zu requests: %.1f sequences/s (%.3f ms per batch per device)\n", a.devices, a.requests, ids.size(),
                    (double)a.devices * a.requests * (double)ids.size() / sec, 1e3 * sec / a.requests);
    }
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
}
