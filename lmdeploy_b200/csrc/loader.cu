// Loader for TurboMind workspaces: reads the per-rank binary files that lmdeploy's deploy.py writes
// and that LlamaWeight::loadModel / LlamaDecoderLayerWeight::loadModel read
// (src/turbomind/models/llama/LlamaWeight.cc:86-106, LlamaDecoderLayerWeight.cc:113-222,261-307),
// int4 (W4A16) path only, already sliced per tensor-parallel rank:
//
//   <dir>/tok_embeddings.weight                       half [vocab, hidden]
//   <dir>/norm.weight                                 half [hidden]
//   <dir>/output.weight                               half [vocab, hidden]      (this rank uses its vocab / tp rows)
//   <dir>/layers.<l>.attention_norm.weight            half [hidden]
//   <dir>/layers.<l>.ffn_norm.weight                  half [hidden]
//   <dir>/layers.<l>.<w>.<rank>.qweight               int32 runtime int4 layout, K * N / 8 words
//   <dir>/layers.<l>.<w>.<rank>.scales_zeros          half2 {64 + z, s}, [K / group, N]
//       for <w> in attention.w_qkv, attention.wo, feed_forward.w13, feed_forward.w2
//   <dir>/layers.<l>.attention.w_qkv.<rank>.bias      half [N]                  (optional)
//   <dir>/layers.<l>.past_kv_scale.<rank>.weight      float [4]                 (optional)
//
// The model owns the device copies (freed by tm_llama_destroy).
#include "llama.h"
#include "tm_b200.h"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

// file -> host buffer of exactly `bytes` bytes; false when missing or of another size
bool read_exact(const std::string& path, size_t bytes, std::vector<unsigned char>& buf, bool* missing)
{
    if (missing) *missing = false;
    std::FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) {
        if (missing) *missing = true;
        return false;
    }
    std::fseek(f, 0, SEEK_END);
    const long size = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    bool ok = size >= 0 && (size_t)size == bytes;
    if (ok) {
        buf.resize(bytes);
        ok = std::fread(buf.data(), 1, bytes, f) == bytes;
    }
    std::fclose(f);
    return ok;
}

struct Uploader {
    tm_llama*                  m;
    int                        rc = TM_OK;
    std::vector<unsigned char> host;

    // whole file (or the byte range [offset, offset + bytes) of a file of `file_bytes`) -> owned device memory
    const void* file(const std::string& path, size_t bytes, size_t file_bytes = 0, size_t offset = 0, bool optional = false)
    {
        if (rc != TM_OK) return nullptr;
        bool missing = false;
        if (!read_exact(path, file_bytes ? file_bytes : bytes, host, &missing)) {
            if (!(optional && missing)) rc = TM_ERR_IO;
            return nullptr;
        }
        void* d = nullptr;
        if (cudaMalloc(&d, bytes) != cudaSuccess) {
            rc = TM_ERR_CUDA;
            return nullptr;
        }
        m->owned.push_back(d);
        if (cudaMemcpy(d, host.data() + offset, bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
            rc = TM_ERR_CUDA;
            return nullptr;
        }
        return d;
    }
};

}  // namespace

extern "C" int tm_llama_load_workspace(tm_llama* m, const char* dir)
{
    if (!m || !dir) return TM_ERR_INVALID_ARG;
    const tm_llama_config& c    = m->cfg;
    const std::string      root = std::string(dir) + "/";
    const std::string      rank = std::to_string(c.tensor_para_rank);
    const size_t           hid  = (size_t)m->hidden;
    int                    prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(m->h->device);
    Uploader up{m};

    // ---- LlamaWeight.cc:91-101
    const void* emb  = up.file(root + "tok_embeddings.weight", (size_t)c.vocab_size * hid * 2);
    const void* norm = up.file(root + "norm.weight", hid * 2);
    const size_t head_rows = (size_t)m->local_vocab;
    const void*  head      = up.file(root + "output.weight", head_rows * hid * 2, (size_t)c.vocab_size * hid * 2,
                               head_rows * c.tensor_para_rank * hid * 2);
    if (up.rc == TM_OK) up.rc = tm_llama_set_globals(m, emb, norm, head);

    // ---- LlamaDecoderLayerWeight.cc:261-307
    struct Lin {
        const char* name;
        size_t      k, n;
    };
    const size_t g       = (size_t)c.group_size;
    const Lin    lins[4] = {{"attention.w_qkv", hid, (size_t)(m->local_heads + 2 * m->local_kv_heads) * 128},
                            {"attention.wo", (size_t)m->local_heads * 128, hid},
                            {"feed_forward.w13", hid, 2 * (size_t)m->local_inter},
                            {"feed_forward.w2", (size_t)m->local_inter, hid}};
    for (int l = 0; l < c.num_layer && up.rc == TM_OK; ++l) {
        const std::string      p = root + "layers." + std::to_string(l) + ".";
        tm_llama_layer_weights w{};
        w.self_attn_norm = up.file(p + "attention_norm.weight", hid * 2);
        w.ffn_norm       = up.file(p + "ffn_norm.weight", hid * 2);
        const void* qw[4];
        const void* sz[4];
        for (int i = 0; i < 4; ++i) {
            const std::string q = p + lins[i].name + "." + rank;
            qw[i]               = up.file(q + ".qweight", lins[i].k * lins[i].n / 2);                 // :214-215
            sz[i]               = up.file(q + ".scales_zeros", lins[i].k / g * lins[i].n * 4);        // :217-219
        }
        w.qkv_qweight = qw[0], w.qkv_scales_zeros = sz[0];
        w.o_qweight = qw[1], w.o_scales_zeros = sz[1];
        w.w13_qweight = qw[2], w.w13_scales_zeros = sz[2];
        w.w2_qweight = qw[3], w.w2_scales_zeros = sz[3];
        w.qkv_bias = up.file(p + lins[0].name + "." + rank + ".bias", lins[0].n * 2, 0, 0, true);
        // :296-306: four floats, or the identity when the file is absent
        w.past_kv_scale[0] = 1.f, w.past_kv_scale[1] = 0.f, w.past_kv_scale[2] = 1.f, w.past_kv_scale[3] = 0.f;
        if (up.rc == TM_OK) {
            bool missing = false;
            if (read_exact(p + "past_kv_scale." + rank + ".weight", 16, up.host, &missing)) {
                std::memcpy(w.past_kv_scale, up.host.data(), 16);
            }
            else if (!missing) {
                up.rc = TM_ERR_IO;
            }
        }
        if (up.rc == TM_OK) up.rc = tm_llama_set_layer(m, l, &w);
    }
    cudaSetDevice(prev);
    return up.rc;
}

// ---------------------------------------------------------------------------------------------
// config.ini of a TurboMind workspace: the [llama] section that lmdeploy/serve/turbomind/deploy.py:209-239
// writes and LlamaTritonModel<T>::LlamaTritonModel reads (src/turbomind/triton_backend/llama/
// LlamaTritonModel.cc:118-143), with the defaults of handleMissingParams (:59-98).
namespace {

std::string trimmed(const std::string& s)
{
    const size_t a = s.find_first_not_of(" \t\r\n");
    if (a == std::string::npos) return "";
    const size_t b = s.find_last_not_of(" \t\r\n");
    return s.substr(a, b - a + 1);
}

struct IniSection {
    std::vector<std::pair<std::string, std::string>> kv;
    bool                                             found = false;

    const std::string* get(const char* key) const
    {
        for (const auto& e : kv) {
            if (e.first == key) return &e.second;
        }
        return nullptr;
    }
    // false when the key is absent and no default was given, or the value does not parse
    bool integer(const char* key, int* out, const int* dflt) const
    {
        const std::string* v = get(key);
        if (!v) {
            if (!dflt) return false;
            *out = *dflt;
            return true;
        }
        char*      end = nullptr;
        const long x   = std::strtol(v->c_str(), &end, 0);
        if (end == v->c_str() || *end) return false;
        *out = (int)x;
        return true;
    }
    bool real(const char* key, float* out, const float* dflt) const
    {
        const std::string* v = get(key);
        if (!v) {
            if (!dflt) return false;
            *out = *dflt;
            return true;
        }
        char*        end = nullptr;
        const double x   = std::strtod(v->c_str(), &end);
        if (end == v->c_str() || *end) return false;
        *out = (float)x;
        return true;
    }
};

IniSection read_ini_section(const std::string& path, const char* section)
{
    IniSection  out;
    std::FILE*  f = std::fopen(path.c_str(), "rb");
    if (!f) return out;
    std::string text;
    char        buf[4096];
    size_t      n;
    while ((n = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    std::fclose(f);
    bool   in_section = false;
    size_t pos        = 0;
    while (pos <= text.size()) {
        size_t eol = text.find('\n', pos);
        if (eol == std::string::npos) eol = text.size();
        const std::string line = trimmed(text.substr(pos, eol - pos));
        pos                    = eol + 1;
        if (line.empty() || line[0] == ';' || line[0] == '#') continue;
        if (line[0] == '[') {
            const size_t close = line.find(']');
            in_section         = close != std::string::npos && trimmed(line.substr(1, close - 1)) == section;
            out.found          = out.found || in_section;
            continue;
        }
        if (!in_section) continue;
        size_t sep = line.find('=');
        if (sep == std::string::npos) sep = line.find(':');
        if (sep == std::string::npos) continue;
        out.kv.emplace_back(trimmed(line.substr(0, sep)), trimmed(line.substr(sep + 1)));
    }
    return out;
}

}  // namespace

extern "C" int tm_llama_read_config(const char* dir, tm_llama_config* cfg, tm_llama_workspace_info* info)
{
    if (!dir || !cfg) return TM_ERR_INVALID_ARG;
    const IniSection s = read_ini_section(std::string(dir) + "/config.ini", "llama");
    if (!s.found) return TM_ERR_IO;
    tm_llama_workspace_info x{};
    const int   zero = 0, one = 1;
    const float theta = 10000.f;
    bool ok = true;
    // required keys (LlamaTritonModel.cc:118-127: no default given there)
    ok = ok && s.integer("head_num", &cfg->head_num, nullptr) && s.integer("size_per_head", &cfg->size_per_head, nullptr)
         && s.integer("inter_size", &cfg->inter_size, nullptr) && s.integer("num_layer", &cfg->num_layer, nullptr)
         && s.integer("vocab_size", &cfg->vocab_size, nullptr) && s.real("norm_eps", &cfg->norm_eps, nullptr)
         && s.integer("start_id", &x.start_id, nullptr) && s.integer("end_id", &x.end_id, nullptr)
         && s.integer("rotary_embedding", &x.rotary_embedding_dim, nullptr);
    // optional keys and their defaults (:120, :128-142)
    ok = ok && s.integer("kv_head_num", &cfg->kv_head_num, &zero) && s.integer("max_batch_size", &cfg->max_batch_size, &zero)
         && s.integer("max_context_token_num", &x.max_context_token_num, &zero) && s.integer("session_len", &cfg->session_len, &zero)
         && s.integer("step_length", &x.step_length, &zero) && s.integer("cache_max_entry_count", &x.cache_max_entry_count, &zero)
         && s.integer("use_context_fmha", &x.use_context_fmha, &one) && s.integer("cache_chunk_size", &x.cache_chunk_size, &zero)
         && s.integer("attn_bias", &x.attn_bias, &zero) && s.integer("quant_policy", &cfg->quant_policy, &zero)
         && s.integer("group_size", &cfg->group_size, &zero) && s.real("rope_theta", &cfg->rope_theta, &theta)
         && s.integer("max_position_embeddings", &x.max_position_embeddings, &zero)
         && s.integer("use_dynamic_ntk", &x.use_dynamic_ntk, &zero) && s.integer("use_logn_attn", &x.use_logn_attn, &zero)
         && s.integer("tensor_para_size", &cfg->tensor_para_size, &one);
    if (!ok) return TM_ERR_INVALID_ARG;
    cfg->tensor_para_rank = 0;
    // handleMissingParams (:59-98)
    if (cfg->kv_head_num == 0) cfg->kv_head_num = cfg->head_num;
    if (cfg->max_batch_size == 0) cfg->max_batch_size = 32;
    if (cfg->session_len == 0) cfg->session_len = 2160;
    if (x.max_context_token_num == 0) {
        int r = 1;
        while ((r + 1) * (r + 1) <= cfg->max_batch_size) ++r;  // (int)std::sqrt(max_batch_size)
        x.max_context_token_num = r;
    }
    if (x.step_length == 0) x.step_length = 1;
    if (x.cache_max_entry_count == 0) x.cache_max_entry_count = 32;
    if (x.cache_chunk_size == 0) x.cache_chunk_size = x.cache_max_entry_count;
    if (x.max_context_token_num <= cfg->max_batch_size) x.max_context_token_num *= cfg->session_len;  // :146-148
    if (const std::string* v = s.get("model_name")) std::snprintf(x.model_name, sizeof(x.model_name), "%s", v->c_str());
    if (const std::string* v = s.get("weight_type")) std::snprintf(x.weight_type, sizeof(x.weight_type), "%s", v->c_str());
    if (info) *info = x;
    return TM_OK;
}
