// Test tooling, not engine code: runs dynalm-project/dynalm's own CPU Transformer on a model
// folder (config.json + model.safetensors holding F32 tensors) and writes the fp32 logits of
// every position of one whole prompt. Built and run by make_golden.py against a CPU build of
// the reference; the engine never links this file.
//
// usage: ref_harness MODEL_DIR OUT.f32 tok0 tok1 ...
#include <cstdio>
#include <cstdlib>
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

using namespace dynalm;

#define DIE_IF(st, what)                                                     \
  do {                                                                       \
    if (!(st).ok()) {                                                        \
      std::fprintf(stderr, "%s: %s\n", what, (st).to_string().c_str());      \
      return 1;                                                              \
    }                                                                        \
  } while (0)

int main(int argc, char** argv) {
  if (argc < 4) {
    std::fprintf(stderr, "usage: ref_harness MODEL_DIR OUT.f32 tok...\n");
    return 2;
  }
  const std::string dir = argv[1];
  std::vector<TokenId> toks;
  for (int i = 3; i < argc; ++i) toks.push_back(static_cast<TokenId>(std::atoi(argv[i])));

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
    if (!hf::parse_tensor_name(info.name, c.architecture, role, layer)) {
      std::fprintf(stderr, "unmapped tensor %s\n", info.name.c_str());
      return 1;
    }
    auto t = (*file)->load_tensor(info);
    DIE_IF(t.status(), info.name.c_str());
    DIE_IF(w.add(role, layer, *t), info.name.c_str());
  }
  DIE_IF(hf::apply_conventions(*cfg, c, w), "apply_conventions");
  const ModelArchitecture* a = find_architecture(c.architecture);
  if (!a) return 1;
  DIE_IF(a->configure(c, w), "configure");
  DIE_IF(a->validate(c, w), "validate");

  ThreadPool pool(2);
  CpuDevice dev(pool, select_best_isa(cpu_info().features));
  const int64_t n = static_cast<int64_t>(toks.size());
  auto tf = Transformer::create(c, w, dev, /*max_batch_tokens=*/n + 16, /*context=*/c.context_length);
  DIE_IF(tf.status(), "Transformer::create");
  // fp32 everywhere: no int8 activation rows, F32 KV.
  KernelPlan base = KernelPlan::defaults();
  base.int8_decode_max_rows = 0;
  (*tf)->set_kernel_base(base);
  auto kv = KvBlockPool::create(kv_geometry_for(c, DType::kF32, 16, c.context_length), dev);
  DIE_IF(kv.status(), "KvBlockPool");

  std::vector<float> logits(static_cast<size_t>(n * c.vocab_size));
  KvBlockTable table(**kv);
  DIE_IF(table.reserve(n), "reserve");
  SeqBatch b{toks, 0, table.block_table(), true};
  b.logits_last = static_cast<int32_t>(n);
  DIE_IF((*tf)->forward_batch({&b, 1}, **kv, logits), "forward_batch");

  std::FILE* f = std::fopen(argv[2], "wb");
  if (!f) return 1;
  std::fwrite(logits.data(), sizeof(float), logits.size(), f);
  std::fclose(f);
  std::printf("device %s, %lld tokens, vocab %lld, tied %d\n", std::string(dev.name()).c_str(),
              static_cast<long long>(n), static_cast<long long>(c.vocab_size), static_cast<int>(c.tied_embeddings));
  return 0;
}
