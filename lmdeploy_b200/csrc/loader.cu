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
