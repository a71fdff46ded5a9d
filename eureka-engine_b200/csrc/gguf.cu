// gguf.cu -- read a Qwen3.5 / Qwen3.5-MoE GGUF file in place: the header becomes the engine's index text
// (the "#cfg" keys and tensor lines a pack directory's index.tsv holds), the file itself, mapped read-only,
// is the pack the tensors are uploaded from.  Host code only.
//
// What it follows in the reference: the key mapping and defaults of tools/gguf2pack.c:541-600 (build_config),
// the tensor naming of its packs (GGUF names kept, tied head = alias of token_embd.weight), Q8_0 re-sliced from
// GGUF's [f16 d][32 x int8] blocks to the pack's row-split [cols x int8][cols/32 x f16] (tools/gguf2pack.c:25-27;
// done at upload, engine.cu: load_tensor), nextn (MTP) blocks counted in block_count, listed after the trunk's and
// not part of it (reports/cuda-moe/scripts/gen_moe.py:56,70).  The GGUF container itself (v2 / v3: magic, counts, typed
// key-values, tensor infos, aligned data section) is read as its public specification describes it.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "host.cuh"
#include "gguf.cuh"

namespace {
struct Rd {
  const uint8_t *p, *end;
  bool bad = false;
  template <class T> T get() {
    T v{};
    if (p + sizeof(T) > end) { bad = true; return v; }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    if (bad || n > (uint64_t)(end - p)) { bad = true; return std::string(); }
    std::string s((const char *)p, (size_t)n);
    p += n;
    return s;
  }
};
struct Val { bool is_num = false, is_str = false; double num = 0; std::string s; uint64_t arr_n = 0; };

// size of a scalar GGUF value type; 0 for strings and arrays
size_t scalar_size(uint32_t t) {
  switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
  }
}
bool read_value(Rd &r, uint32_t t, Val &v) {
  switch (t) {
    case 0: v.num = r.get<uint8_t>(); break;
    case 1: v.num = r.get<int8_t>(); break;
    case 2: v.num = r.get<uint16_t>(); break;
    case 3: v.num = r.get<int16_t>(); break;
    case 4: v.num = r.get<uint32_t>(); break;
    case 5: v.num = r.get<int32_t>(); break;
    case 6: v.num = r.get<float>(); break;
    case 7: v.num = r.get<uint8_t>(); break;
    case 10: v.num = (double)r.get<uint64_t>(); break;
    case 11: v.num = (double)r.get<int64_t>(); break;
    case 12: v.num = r.get<double>(); break;
    case 8: v.s = r.str(); v.is_str = true; return !r.bad;
    case 9: {
      const uint32_t et = r.get<uint32_t>();
      const uint64_t n = r.get<uint64_t>();
      v.arr_n = n;
      if (et == 8) { for (uint64_t i = 0; i < n && !r.bad; i++) r.str(); }
      else if (et == 9) return false;   // nested arrays: not in these files
      else {
        const size_t es = scalar_size(et);
        if (!es || n > (uint64_t)(r.end - r.p) / es) return false;
        r.p += n * es;
      }
      return !r.bad;
    }
    default: return false;
  }
  v.is_num = true;
  return !r.bad;
}
}  // namespace

void gguf_unmap(GgufFile &g) {
  if (g.map) munmap((void *)g.map, g.size);
  if (g.fd >= 0) close(g.fd);
  g.map = nullptr; g.fd = -1; g.size = 0;
}

int gguf_map(const char *path, GgufFile &g) {
  g.fd = open(path, O_RDONLY);
  if (g.fd < 0) return llb_fail("gguf: cannot open %s", path);
  struct stat st;
  if (fstat(g.fd, &st) || st.st_size < 32) { gguf_unmap(g); return llb_fail("gguf: %s is not a GGUF file", path); }
  g.size = (size_t)st.st_size;
  void *mp = mmap(nullptr, g.size, PROT_READ, MAP_PRIVATE, g.fd, 0);
  if (mp == MAP_FAILED) { g.map = nullptr; gguf_unmap(g); return llb_fail("gguf: cannot map %s", path); }
  g.map = (const uint8_t *)mp;
  Rd r{g.map, g.map + g.size};
  if (memcmp(g.map, "GGUF", 4)) { gguf_unmap(g); return llb_fail("gguf: %s has no GGUF magic", path); }
  r.p += 4;
  const uint32_t ver = r.get<uint32_t>();
  const uint64_t nt = r.get<uint64_t>(), nkv = r.get<uint64_t>();
  if (ver < 2 || ver > 3 || nt > (1u << 20) || nkv > (1u << 20)) { gguf_unmap(g); return llb_fail("gguf: version %u with %llu tensors", ver, (unsigned long long)nt); }
  std::map<std::string, Val> kv;
  for (uint64_t i = 0; i < nkv; i++) {
    std::string key = r.str();
    const uint32_t t = r.get<uint32_t>();
    Val v;
    if (r.bad || !read_value(r, t, v)) { gguf_unmap(g); return llb_fail("gguf: bad key-value %llu (%s)", (unsigned long long)i, key.c_str()); }
    kv[key] = v;
  }
  struct TI { std::string name; uint64_t ne[4]; uint32_t nd, type; uint64_t off; };
  std::vector<TI> tis((size_t)nt);
  for (auto &t : tis) {
    t.name = r.str();
    t.nd = r.get<uint32_t>();
    if (r.bad || t.nd < 1 || t.nd > 4) { gguf_unmap(g); return llb_fail("gguf: tensor %s has %u dimensions", t.name.c_str(), t.nd); }
    for (uint32_t d = 0; d < 4; d++) t.ne[d] = d < t.nd ? r.get<uint64_t>() : 1;
    t.type = r.get<uint32_t>();
    t.off = r.get<uint64_t>();
  }
  if (r.bad) { gguf_unmap(g); return llb_fail("gguf: truncated header"); }
  uint64_t align = 32;
  if (kv.count("general.alignment") && kv["general.alignment"].is_num) align = (uint64_t)kv["general.alignment"].num;
  if (align < 1 || (align & (align - 1))) { gguf_unmap(g); return llb_fail("gguf: alignment %llu", (unsigned long long)align); }
  const uint64_t data0 = ((uint64_t)(r.p - g.map) + align - 1) / align * align;

  // ---- configuration (tools/gguf2pack.c:541-600) ----
  if (!kv.count("general.architecture") || !kv["general.architecture"].is_str) { gguf_unmap(g); return llb_fail("gguf: no general.architecture"); }
  const std::string arch = kv["general.architecture"].s;
  if (arch != "qwen35" && arch != "qwen35moe" && arch != "clef") { gguf_unmap(g); return llb_fail("gguf: architecture %s is not the Qwen3.5 hybrid", arch.c_str()); }
  bool miss = false;
  std::string missing;
  auto num = [&](const char *k, bool need, double dflt) -> double {
    auto it = kv.find(arch + "." + k);
    if (it == kv.end() || !it->second.is_num) { if (need) { miss = true; missing = k; } return dflt; }
    return it->second.num;
  };
  const bool moe = arch == "qwen35moe";
  const long long blocks = (long long)num("block_count", true, 0), nextn = (long long)num("nextn_predict_layers", false, 0);
  const long long H = (long long)num("attention.head_count", true, 0), KV = (long long)num("attention.head_count_kv", true, 0);
  const long long d = (long long)num("embedding_length", true, 0), hd = (long long)num("attention.key_length", true, 0);
  const long long ef = moe ? (long long)num("expert_feed_forward_length", true, 0) : 0, sf = moe ? (long long)num("expert_shared_feed_forward_length", true, 0) : 0;
  const long long f = moe ? (ef > sf ? ef : sf) : (long long)num("feed_forward_length", true, 0);
  const double rope_base = num("rope.freq_base", false, 10000.0), eps = num("attention.layer_norm_rms_epsilon", true, 0);
  const long long rope_dim = (long long)num("rope.dimension_count", false, (double)hd), interval = (long long)num("full_attention_interval", true, 0);
  const long long KC = (long long)num("ssm.conv_kernel", true, 0), SZ = (long long)num("ssm.state_size", true, 0), GK = (long long)num("ssm.group_count", true, 0);
  const long long TR = (long long)num("ssm.time_step_rank", true, 0), inner = (long long)num("ssm.inner_size", true, 0);
  const long long ne = moe ? (long long)num("expert_count", true, 0) : 0, nk = moe ? (long long)num("expert_used_count", true, 0) : 0;
  if (miss) { gguf_unmap(g); return llb_fail("gguf: key %s.%s is missing", arch.c_str(), missing.c_str()); }
  const TI *embd = nullptr, *outw = nullptr;
  for (const auto &t : tis) { if (t.name == "token_embd.weight") embd = &t; if (t.name == "output.weight") outw = &t; }
  if (!embd) { gguf_unmap(g); return llb_fail("gguf: no token_embd.weight"); }
  long long V = (long long)num("vocab_size", false, 0);
  if (V <= 0) V = kv.count("tokenizer.ggml.tokens") ? (long long)kv["tokenizer.ggml.tokens"].arr_n : 0;
  if (V <= 0) V = (long long)embd->ne[1];
  const long long L = blocks - nextn;
  char buf[512];
  std::string &ix = g.index;
  ix.clear();
  auto cfg = [&](const char *k, long long v) { snprintf(buf, sizeof buf, "#cfg\t%s\t%lld\n", k, v); ix += buf; };
  cfg("n_layers", L); cfg("n_heads", H); cfg("n_kv_heads", KV); cfg("d_model", d); cfg("head_dim", hd); cfg("d_ff", f); cfg("vocab_size", V);
  cfg("full_attention_interval", interval); cfg("ssm_conv_kernel", KC); cfg("ssm_state_size", SZ); cfg("ssm_group_count", GK);
  cfg("ssm_time_step_rank", TR); cfg("ssm_inner_size", inner); cfg("linear_key_dim", SZ * GK); cfg("linear_value_head_dim", TR > 0 ? inner / TR : 0);
  cfg("linear_conv_dim", 2 * SZ * GK + inner); cfg("rope_dim", rope_dim);
  snprintf(buf, sizeof buf, "#cfg\trope_freq_base\t%.9g\n#cfg\trms_norm_eps\t%.9g\n", rope_base, eps); ix += buf;
  if (moe) { cfg("expert_count", ne); cfg("expert_used_count", nk); cfg("expert_feed_forward_length", ef); cfg("expert_shared_feed_forward_length", sf); }
  g.nextn = (int)nextn;

  // ---- tensors: absolute file offsets; rows = product of the outer dimensions ----
  auto line = [&](const std::string &name, const TI &t) -> int {
    const char *ty = nullptr;
    uint64_t bb = 0, be = 1;   // bytes per block, elements per block
    switch (t.type) {
      case 0: ty = "F32"; bb = 4; be = 1; break;
      case 8: ty = "Q8_0G"; bb = 34; be = 32; break;      // GGUF's blocked Q8_0: re-sliced at upload
      case 12: ty = "Q4_K"; bb = 144; be = 256; break;
      case 13: ty = "Q5_K"; bb = 176; be = 256; break;
      case 14: ty = "Q6_K"; bb = 210; be = 256; break;
      default: return llb_fail("gguf: tensor %s has ggml type %u; F32, Q8_0, Q4_K, Q5_K, Q6_K are read", name.c_str(), t.type);
    }
    const uint64_t cols = t.ne[0], rows = t.ne[1] * t.ne[2] * t.ne[3];
    if (cols % be) return llb_fail("gguf: tensor %s: %llu columns are not whole blocks", name.c_str(), (unsigned long long)cols);
    const uint64_t nb = rows * (cols / be) * bb, off = data0 + t.off;
    if (off + nb > g.size) return llb_fail("gguf: tensor %s reaches past the end of the file", name.c_str());
    if (rows > 0x7fffffffull || cols > 0x7fffffffull) return llb_fail("gguf: tensor %s is too large", name.c_str());
    snprintf(buf, sizeof buf, "%s\t%llu\t%llu\t%llu\t%llu\t%s\n", name.c_str(), (unsigned long long)off, (unsigned long long)nb,
             (unsigned long long)rows, (unsigned long long)cols, ty);
    ix += buf;
    return 0;
  };
  for (const auto &t : tis) {
    // only what the path reads: the blocks (the trunk's, and a nextn block after them, which the engine takes as
    // its drafter), the embedding, the head and its norm (tokenizer-side and vision tensors stay in the file)
    long long il = -1;
    if (t.name.rfind("blk.", 0) == 0) il = atoll(t.name.c_str() + 4);
    const bool want = (il >= 0 && il < blocks) || t.name == "token_embd.weight" || t.name == "output.weight" || t.name == "output_norm.weight";
    if (!want) continue;
    if (line(t.name, t)) { gguf_unmap(g); return -1; }
  }
  if (!outw && line("output.weight", *embd)) { gguf_unmap(g); return -1; }   // tied head
  return 0;
}
