// model_registry.cpp -- see model_registry.h.
#include "model_registry.h"

#include <dirent.h>
#include <stdio.h>
#include <stdlib.h>
#include <unistd.h>

#include <algorithm>
#include <vector>

#include "checkpoint.h"
#include "json_min.h"

namespace qie {
namespace {

struct Row {
  const char* architecture;
  int family;
};
const Row kRegistry[] = {
    {"Nogatar", FAMILY_NOGATAR},
    {"Fosavik", FAMILY_FOSAVIK},
    {"Ditenex", FAMILY_DITENEX},
    {"Dedunex", FAMILY_DEDUNEX},
    {"Qwen2ForCausalLM", FAMILY_QWEN},
    {"Qwen3ForCausalLM", FAMILY_QWEN},
};

bool slurp(const std::string& path, std::string* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  char buf[65536];
  size_t n;
  out->clear();
  while ((n = fread(buf, 1, sizeof buf, f)) > 0) out->append(buf, n);
  fclose(f);
  return true;
}

}  // namespace

const char* registry_names() {
  static const std::string names = [] {
    std::string s;
    for (const Row& r : kRegistry) s += (s.empty() ? "" : ",") + std::string(r.architecture);
    return s;
  }();
  return names.c_str();
}

int registry_family_of_config(const std::string& text, std::string* arch, std::string* err) {
  JsonValue root;
  std::string perr;
  if (!JsonReader::parse(text.data(), text.data() + text.size(), &root, &perr)) {
    if (err) *err = "config.json: " + perr;
    return -1;
  }
  std::string name;
  if (const JsonValue* a = root.have("architecture")) name = a->str;
  else if (const JsonValue* as = root.have("architectures"))
    if (as->kind == JsonValue::Array && !as->arr.empty()) name = as->arr[0].str;
  if (arch) *arch = name;
  for (const Row& r : kRegistry)
    if (name == r.architecture) return r.family;
  if (err) *err = "config.json: architecture '" + name + "' is not registered (known: " + registry_names() + ")";
  return -1;
}

int registry_family_of_dir(const std::string& dir, std::string* arch, std::string* err) {
  std::string text;
  if (!slurp(dir + "/config.json", &text)) {
    if (err) *err = "cannot read " + dir + "/config.json";
    return -1;
  }
  return registry_family_of_config(text, arch, err);
}

std::string registry_convert_qwen_dir(const std::string& dir, std::string* meta_path, std::string* weights_path) {
  std::vector<std::string> shards;
  if (DIR* d = opendir(dir.c_str())) {
    while (dirent* ent = readdir(d)) {
      const std::string n = ent->d_name;
      if (n.size() > 12 && n.compare(n.size() - 12, 12, ".safetensors") == 0) shards.push_back(dir + "/" + n);
    }
    closedir(d);
  }
  if (shards.empty()) return "no .safetensors file in " + dir;
  std::sort(shards.begin(), shards.end());
  const char* tmp = getenv("TMPDIR");
  std::string tmpl = std::string(tmp && *tmp ? tmp : "/tmp") + "/qie_convert_XXXXXX";
  std::vector<char> buf(tmpl.begin(), tmpl.end());
  buf.push_back('\0');
  if (!mkdtemp(buf.data())) return "cannot create a temporary folder under " + tmpl;
  *meta_path = std::string(buf.data()) + "/meta_data.txt";
  *weights_path = std::string(buf.data()) + "/weights.bin";
  size_t total = 0;
  int n = 0;
  // checkpoints without an lm_head tensor tie it to the embedding
  return convert_safetensors(shards, *meta_path, *weights_path, true, &total, &n);
}

}  // namespace qie
