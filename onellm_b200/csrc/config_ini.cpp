// Reads the config.ini that the reference's converter writes beside the weight files
// (tools/FT_convert_weight_to_bin_final.py:43-64: a [llama] section with head_num, kv_head_num, hidden_size,
// head_size, inter_size, num_layer, vocab_size, bos_token_id, eos_token_id, weight_data_type,
// max_position_embeddings, rope_theta, rms_norm_eps, attention_bias, top_k) into the model configuration.
// The reference itself never reads the file back (its model class is an outline, src/models/llama/llama.cpp:1-32).
#include <ctype.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>

#include "common.cuh"

namespace onellm {

static std::string trim(const std::string& s)
{
    size_t a = 0, b = s.size();
    while (a < b && isspace((unsigned char)s[a])) a++;
    while (b > a && isspace((unsigned char)s[b - 1])) b--;
    return s.substr(a, b - a);
}

static std::string lower(std::string s)
{
    for (auto& c : s) c = (char)tolower((unsigned char)c);
    return s;
}

// key -> value of the [llama] section (keys lower-cased, as Python's configparser writes them)
static int read_section(const char* path, std::map<std::string, std::string>& kv)
{
    FILE* f = fopen(path, "r");
    ONELLM_REQUIRE(f, ONELLM_ERR_IO, "cannot open %s", path);
    char line[1024];
    bool in_section = false, seen = false;
    while (fgets(line, sizeof(line), f)) {
        const std::string s = trim(line);
        if (s.empty() || s[0] == '#' || s[0] == ';') continue;
        if (s[0] == '[') {
            in_section = lower(s) == "[llama]";
            seen |= in_section;
            continue;
        }
        if (!in_section) continue;
        size_t eq = s.find('=');
        const size_t colon = s.find(':');
        if (eq == std::string::npos || (colon != std::string::npos && colon < eq)) eq = colon;  // "key: value" is valid too
        if (eq == std::string::npos) continue;
        kv[lower(trim(s.substr(0, eq)))] = trim(s.substr(eq + 1));
    }
    fclose(f);
    ONELLM_REQUIRE(seen, ONELLM_ERR_IO, "%s has no [llama] section", path);
    return ONELLM_OK;
}

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_llama_config_from_ini(const char* path, onellm_llama_config* cfg, int* top_k)
{
    ONELLM_REQUIRE(path && cfg, ONELLM_ERR_ARG, "llama_config_from_ini: null pointer");
    std::map<std::string, std::string> kv;
    const int rc = read_section(path, kv);
    if (rc) return rc;
    bool bad = false;
    std::string bad_key;
    auto integer = [&](const char* key, int* out, bool required) {
        auto it = kv.find(key);
        if (it == kv.end()) {
            if (required && !bad) {
                bad = true;
                bad_key = std::string("missing key ") + key;
            }
            return;
        }
        char* end = nullptr;
        const long v = strtol(it->second.c_str(), &end, 10);
        if (end == it->second.c_str() || *end != '\0') {
            if (!bad) {
                bad = true;
                bad_key = std::string(key) + " = " + it->second + " is not an integer";
            }
            return;
        }
        *out = (int)v;
    };
    auto real = [&](const char* key, float* out) {
        auto it = kv.find(key);
        if (it == kv.end()) return;
        char* end = nullptr;
        const double v = strtod(it->second.c_str(), &end);
        if (end == it->second.c_str() || *end != '\0') {
            if (!bad) {
                bad = true;
                bad_key = std::string(key) + " = " + it->second + " is not a number";
            }
            return;
        }
        *out = (float)v;
    };
    int hidden = 0, max_pos = 0;
    integer("head_num", &cfg->head_num, true);
    integer("kv_head_num", &cfg->kv_head_num, true);
    integer("head_size", &cfg->head_size, true);
    integer("hidden_size", &hidden, false);
    integer("inter_size", &cfg->inter_size, true);
    integer("num_layer", &cfg->num_layers, true);
    integer("vocab_size", &cfg->vocab_size, true);
    integer("bos_token_id", &cfg->bos_id, false);
    integer("eos_token_id", &cfg->eos_id, false);
    integer("max_position_embeddings", &max_pos, false);
    real("rope_theta", &cfg->rope_base);
    real("rms_norm_eps", &cfg->rms_eps);
    if (top_k) integer("top_k", top_k, false);
    auto ab = kv.find("attention_bias");
    if (ab != kv.end()) {
        const std::string v = lower(ab->second);
        if (v == "true" || v == "1" || v == "yes")
            cfg->attn_bias = 1;
        else if (v == "false" || v == "0" || v == "no")
            cfg->attn_bias = 0;
        else if (!bad) {
            bad = true;
            bad_key = "attention_bias = " + ab->second + " is neither True nor False";
        }
    }
    auto wt = kv.find("weight_data_type");
    if (wt != kv.end() && !bad) {
        const std::string v = lower(wt->second);
        if (v != "fp32" && v != "fp16") {  // the loader tells fp32 from fp16 files by their size; nothing else is read
            bad = true;
            bad_key = "weight_data_type = " + wt->second + " (fp32 or fp16)";
        }
    }
    ONELLM_REQUIRE(!bad, ONELLM_ERR_IO, "%s: %s", path, bad_key.c_str());
    cfg->hidden = cfg->head_num * cfg->head_size;
    ONELLM_REQUIRE(hidden == 0 || hidden == cfg->hidden, ONELLM_ERR_IO, "%s: hidden_size %d != head_num %d x head_size %d", path, hidden,
                   cfg->head_num, cfg->head_size);
    if (cfg->max_seq_len <= 0) cfg->max_seq_len = max_pos;  // the caller's cache length wins over the model's position limit
    return ONELLM_OK;
}

extern "C" int onellm_llama_create_from_ini(const char* path, int max_batch, int max_seq_len, int tp_rank, int tp_size, onellm_llama** out)
{
    ONELLM_REQUIRE(path && out, ONELLM_ERR_ARG, "llama_create_from_ini: null pointer");
    onellm_llama_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.max_batch = max_batch;
    cfg.max_seq_len = max_seq_len;
    cfg.tp_rank = tp_rank;
    cfg.tp_size = tp_size < 1 ? 1 : tp_size;
    cfg.bos_id = 1;
    cfg.eos_id = 2;
    int top_k = 0;
    int rc = onellm_llama_config_from_ini(path, &cfg, &top_k);
    if (rc) return rc;
    rc = onellm_llama_create(&cfg, out);
    if (rc) return rc;
    if (top_k >= 1 && top_k <= 64) rc = onellm_llama_set_sampling(*out, top_k, 1.0f, 0);
    return rc;
}
