// The reference arm of bench.py: times dynalm-project/dynalm's own engine, unmodified, on its CPU device
// (the project has no CUDA code of its own; its GPU backends are ggml's, fetched from the network at configure
// time). Everything below is the reference's public C++ API and stock code path:
//   hf::read_config -> SafeTensorsFile::load_tensor -> TensorRegistry -> apply_conventions -> architecture
//   configure/validate -> Transformer::create on CpuDevice -> KvBlockPool -> forward_batch -> sample_greedy,
// and for the end-to-end figure the stock Scheduler (submit / step / token callbacks).
// Nothing of dynalm_b200 is linked or called. Built by baseline/build_reference.sh against a CPU-only build of
// the reference (-DDYNALM_NATIVE_ONLY=ON -DENABLE_SERVER=OFF).
//
// usage: ref_bench MODEL_DIR BATCH HELD STEPS WARMUP PREFILL_TOKENS POINTS(e.g. 1,64 or -) POINT_STEPS THREADS(0 = physical cores)
// prints one JSON object.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <sstream>
#include <string>
#include <vector>

#include "api/json.h"
#include "dynacore/cpu/cpu_device.h"
#include "dynacore/hardware/cpu_info.h"
#include "dynacore/hardware/isa.h"
#include "kv_cache/kv_cache.h"
#include "loader/hf/hf_model.h"
#include "loader/safetensors/safetensors.h"
#include "model/architecture.h"
#include "model/transformer.h"
#include "runtime/sequence.h"
#include "sampling/sampler.h"
#include "scheduler/scheduler.h"
#include "tokenizer/tokenizer.h"

using namespace dynalm;
using Clock = std::chrono::steady_clock;

#define DIE_IF(st, what)                                                      \
  do {                                                                        \
    if (!(st).ok()) {                                                         \
      std::fprintf(stderr, "%s: %s\n", what, (st).to_string().c_str());       \
      return 1;                                                               \
    }                                                                         \
  } while (0)

static double ms_since(Clock::time_point t0) {
  return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}

int main(int argc, char** argv) {
  if (argc < 10) {
    std::fprintf(stderr, "usage: ref_bench MODEL_DIR BATCH HELD STEPS WARMUP PREFILL_TOKENS POINTS POINT_STEPS THREADS\n");
    return 2;
  }
  const std::string dir = argv[1];
  const int batch = std::atoi(argv[2]), held = std::atoi(argv[3]), steps = std::atoi(argv[4]);
  const int warmup = std::atoi(argv[5]), prefill_tokens = std::atoi(argv[6]);
  std::vector<int> batches{batch};
  if (std::string(argv[7]) != "-") {
    std::stringstream ss(argv[7]);
    for (std::string t; std::getline(ss, t, ',');) batches.push_back(std::atoi(t.c_str()));
  }
  const int point_steps = std::max(1, std::atoi(argv[8]));
  int threads = std::atoi(argv[9]);
  if (threads <= 0) threads = cpu_info().physical_cores;
  const int max_b = *std::max_element(batches.begin(), batches.end());

  auto cfg = hf::read_json_file(dir + "/config.json");
  DIE_IF(cfg.status(), "config.json");
  auto mc = hf::read_config(*cfg);
  DIE_IF(mc.status(), "read_config");
  ModelConfig c = *mc;
  auto file = safetensors::SafeTensorsFile::open(dir + "/model.safetensors");
  DIE_IF(file.status(), "safetensors");
  TensorRegistry w(c.num_layers);
  for (const auto& info : (*file)->tensors()) {
    TensorRole role;
    int layer = -1;
    if (!hf::parse_tensor_name(info.name, c.architecture, role, layer)) continue;
    auto t = (*file)->load_tensor(info);
    DIE_IF(t.status(), info.name.c_str());
    DIE_IF(w.add(role, layer, *t), info.name.c_str());
  }
  DIE_IF(hf::apply_conventions(*cfg, c, w), "apply_conventions");
  const ModelArchitecture* a = find_architecture(c.architecture);
  if (!a) return 1;
  DIE_IF(a->configure(c, w), "configure");
  DIE_IF(a->validate(c, w), "validate");

  ThreadPool pool(threads);
  CpuDevice dev(pool, select_best_isa(cpu_info().features));
  const int total_steps = warmup + steps;
  const int max_batch_tokens = std::max(prefill_tokens, 256);
  auto tf = Transformer::create(c, w, dev, max_batch_tokens, c.context_length);
  DIE_IF(tf.status(), "Transformer::create");
  const int64_t per_seq = held + 2 * total_steps + 64;
  auto kv = KvBlockPool::create(kv_geometry_for(c, DType::kF16, 16, (max_b + 1) * per_seq + prefill_tokens), dev);
  DIE_IF(kv.status(), "KvBlockPool");

  std::mt19937 rng(0);
  std::uniform_int_distribution<int> any_token(0, static_cast<int>(c.vocab_size) - 1);
  std::vector<float> logits(static_cast<size_t>(max_b) * static_cast<size_t>(c.vocab_size));

  // ---- prefill of one prompt (also the context every decoding sequence starts from) ----------------------------
  std::vector<TokenId> prompt(static_cast<size_t>(std::max(prefill_tokens, held)));
  for (auto& t : prompt) t = static_cast<TokenId>(any_token(rng));
  double prefill_ms = 0.0;
  KvBlockTable source(**kv);
  {
    // a short untimed pass first: threads started, pages touched
    KvBlockTable warm(**kv);
    DIE_IF(warm.reserve(64), "reserve");
    SeqBatch b{std::span<const TokenId>(prompt.data(), 64), 0, warm.block_table(), true};
    DIE_IF((*tf)->forward_batch({&b, 1}, **kv, std::span<float>(logits.data(), static_cast<size_t>(c.vocab_size))), "warm");
  }
  {
    DIE_IF(source.reserve(prefill_tokens), "reserve");
    SeqBatch b{std::span<const TokenId>(prompt.data(), static_cast<size_t>(prefill_tokens)), 0, source.block_table(), true};
    const auto t0 = Clock::now();
    DIE_IF((*tf)->forward_batch({&b, 1}, **kv, std::span<float>(logits.data(), static_cast<size_t>(c.vocab_size))), "prefill");
    prefill_ms = ms_since(t0);
  }
  if (held > prefill_tokens) {
    std::fprintf(stderr, "HELD must not exceed PREFILL_TOKENS\n");
    return 2;
  }
  source.truncate(held);

  // ---- decode: B sequences of `held` tokens each, one token per sequence and step, greedy ----------------------
  std::string points = "{";
  double ms_main = 0.0;
  for (size_t bi = 0; bi < batches.size(); ++bi) {
    const int B = batches[bi];
    std::vector<KvBlockTable> tables;
    tables.reserve(static_cast<size_t>(B));
    for (int i = 0; i < B; ++i) {
      tables.push_back(source.clone());
      DIE_IF(tables.back().make_writable(0, held), "make_writable");     // every sequence reads its own memory
    }
    std::vector<TokenId> next(static_cast<size_t>(B));
    for (auto& t : next) t = static_cast<TokenId>(any_token(rng));
    std::vector<SeqBatch> seqs(static_cast<size_t>(B));
    auto step = [&](int pos) -> Status {
      for (int i = 0; i < B; ++i) {
        ENGINE_RETURN_IF_ERROR(tables[static_cast<size_t>(i)].reserve(pos + 1));
        ENGINE_RETURN_IF_ERROR(tables[static_cast<size_t>(i)].make_writable(pos, pos + 1));
        seqs[static_cast<size_t>(i)] = SeqBatch{std::span<const TokenId>(&next[static_cast<size_t>(i)], 1), pos,
                                                 tables[static_cast<size_t>(i)].block_table(), true};
      }
      ENGINE_RETURN_IF_ERROR((*tf)->forward_batch(seqs, **kv, std::span<float>(logits.data(), static_cast<size_t>(B) * static_cast<size_t>(c.vocab_size))));
      for (int i = 0; i < B; ++i)
        next[static_cast<size_t>(i)] = sample_greedy(std::span<const float>(logits.data() + static_cast<size_t>(i) * static_cast<size_t>(c.vocab_size), static_cast<size_t>(c.vocab_size)));
      return Status::Ok();
    };
    int pos = held;
    const int n_warm = bi == 0 ? warmup : std::min(warmup, 2), n_steps = bi == 0 ? steps : point_steps;
    for (int s = 0; s < n_warm; ++s) DIE_IF(step(pos++), "decode warm-up");
    const auto t0 = Clock::now();
    for (int s = 0; s < n_steps; ++s) DIE_IF(step(pos++), "decode");
    const double ms = ms_since(t0) / n_steps;
    if (bi == 0) ms_main = ms;
    char buf[96];
    std::snprintf(buf, sizeof(buf), "%s\"%d\": %.4f", bi ? ", " : "", B, ms);
    points += buf;
  }
  points += "}";

  // ---- end to end: the stock Scheduler, token ids in, token callbacks out ------------------------------------------
  double e2e_tokens_per_s = 0.0;
  {
    TokenizerData td;
    td.model = TokenizerData::Model::kBpe;
    td.tokens.reserve(static_cast<size_t>(c.vocab_size));
    for (int64_t i = 0; i < c.vocab_size; ++i) td.tokens.push_back("t" + std::to_string(i));
    auto tok = Tokenizer::create(std::move(td));
    DIE_IF(tok.status(), "Tokenizer::create");
    SchedulerConfig sc;
    sc.decode_token_budget = 64;
    sc.prefill_token_budget = max_batch_tokens - 64;
    sc.max_prefill_chunk = 0;
    sc.max_running = 64;
    Scheduler sched(**tf, **kv, **tok, sc);
    int64_t tokens_out = 0;
    std::vector<int> got(static_cast<size_t>(batch), 0);
    for (int i = 0; i < batch; ++i) {
      Request r;
      r.prompt.resize(static_cast<size_t>(held));
      for (auto& t : r.prompt) t = static_cast<TokenId>(any_token(rng));
      r.stop = StopParams{total_steps + 8, false};
      r.on_event = [&tokens_out, &got, i](const RequestEvent& ev) {
        if (!ev.finished && ev.token != kNoToken) {
          ++tokens_out;
          ++got[static_cast<size_t>(i)];
        }
      };
      sched.submit(std::move(r));
    }
    // untimed: every prompt computed and `warmup` tokens decoded by every request
    auto all_have = [&](int n) { return std::all_of(got.begin(), got.end(), [n](int g) { return g >= n; }); };
    while (!all_have(1 + warmup))
      if (!sched.step()) break;
    const int64_t before = tokens_out;
    const auto t0 = Clock::now();
    for (int s = 0; s < steps; ++s)
      if (!sched.step()) break;
    const double secs = ms_since(t0) * 1e-3;
    e2e_tokens_per_s = static_cast<double>(tokens_out - before) / secs;
  }

  std::printf("{\"device\": \"%s\", \"threads\": %d, \"kv\": \"f16\", \"prefill_ms\": %.3f, \"decode_ms_per_step\": %.4f, "
              "\"points_ms_per_step\": %s, \"e2e_tokens_per_s\": %.2f}\n",
              std::string(dev.name()).c_str(), threads, prefill_ms, ms_main, points.c_str(), e2e_tokens_per_s);
  return 0;
}
