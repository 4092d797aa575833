// model_registry.h -- which model family serves a model folder.  A folder holds config.json (+ safetensors); the
// configuration's "architecture" string (or the first entry of Hugging Face's "architectures" list) is looked up in
// the table of model_registry.cpp.  Adding a family = one row there + its create function in the C ABI.
#pragma once
#include <string>

namespace qie {

enum ModelFamily { FAMILY_QWEN = 0, FAMILY_NOGATAR = 1, FAMILY_FOSAVIK = 2, FAMILY_DITENEX = 3, FAMILY_DEDUNEX = 4 };

// comma-separated architecture names the registry knows
const char* registry_names();
// family id (>= 0) of a configuration text / a model folder; -1 and *err on unknown or unreadable input
int registry_family_of_config(const std::string& config_json, std::string* arch, std::string* err);
int registry_family_of_dir(const std::string& dir, std::string* arch, std::string* err);
// Qwen folders: the safetensors shards of `dir` (model.safetensors, or model-*-of-*.safetensors in name order) are
// converted to a temporary meta_data.txt + weights.bin (the caller removes them after loading); "" or the error
std::string registry_convert_qwen_dir(const std::string& dir, std::string* meta_path, std::string* weights_path);

}  // namespace qie
