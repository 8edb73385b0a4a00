#include <algorithm>
#include "checkpoint.hpp"

#include <cstdio>
#include <cstring>
#include <vector>

namespace mantle {

namespace {
constexpr uint32_t kMagic = 0x42534C54u;  // checkpoint.mojo:26
constexpr uint32_t kVersion = 1u;         // checkpoint.mojo:29
enum : uint8_t { kTensor = 0, kMomentum = 1, kRms = 2 };  // checkpoint.mojo:32-39

struct File {
    FILE* f;
    File(const std::string& path, const char* mode) : f(std::fopen(path.c_str(), mode)) {
        if (!f) throw Error(MTL_ERR_INVALID, "cannot open checkpoint file " + path);
    }
    ~File() { if (f) std::fclose(f); }
};

void put_u32(FILE* f, uint32_t v) {
    unsigned char b[4] = {(unsigned char)(v & 255), (unsigned char)((v >> 8) & 255), (unsigned char)((v >> 16) & 255),
                          (unsigned char)((v >> 24) & 255)};
    if (std::fwrite(b, 1, 4, f) != 4) throw Error(MTL_ERR_INVALID, "checkpoint write failed");
}

uint32_t get_u32(const std::vector<unsigned char>& d, size_t& off) {
    if (off + 4 > d.size()) throw Error(MTL_ERR_INVALID, "checkpoint file is truncated");
    uint32_t v = (uint32_t)d[off] | ((uint32_t)d[off + 1] << 8) | ((uint32_t)d[off + 2] << 16) | ((uint32_t)d[off + 3] << 24);
    off += 4;
    return v;
}

// _write_tensor, checkpoint.mojo:86-116
void put_entry(FILE* f, uint32_t id, uint8_t kind, const TensorShape& shape, const float* host) {
    put_u32(f, id);
    if (std::fwrite(&kind, 1, 1, f) != 1) throw Error(MTL_ERR_INVALID, "checkpoint write failed");
    put_u32(f, (uint32_t)shape.rank);
    for (int i = 0; i < shape.rank; ++i) put_u32(f, (uint32_t)shape.dims[i]);
    const size_t n = (size_t)shape.num_elements();
    if (std::fwrite(host, 4, n, f) != n) throw Error(MTL_ERR_INVALID, "checkpoint write failed");
}
}  // namespace

void save_checkpoint(const std::string& path, const Model& model, const Adam* adam, int iter) {
    File file(path, "wb");
    const std::vector<Symbol>& all = model.allocation_order();
    const std::vector<Symbol>& tr = model.trainable_parameters();
    put_u32(file.f, kMagic);
    put_u32(file.f, kVersion);
    put_u32(file.f, (uint32_t)iter);
    put_u32(file.f, (uint32_t)all.size());
    put_u32(file.f, adam ? (uint32_t)(2 * tr.size()) : 0u);
    std::vector<float> host;
    for (const Symbol& s : all) {
        host.resize((size_t)s.shape.num_elements());
        model.get_tensor(s.id, host.data());
        put_entry(file.f, (uint32_t)s.id, kTensor, s.shape, host.data());
    }
    if (!adam) return;
    std::vector<float> flat((size_t)std::max<int64_t>(model.n_trainable(), 1));
    const std::vector<int64_t>& off = model.trainable_offsets();
    for (int which = 0; which < 2; ++which) {  // all momentum entries, then all rms entries
        adam->get_state(which, flat.data());
        for (size_t p = 0; p < tr.size(); ++p)
            put_entry(file.f, (uint32_t)tr[p].id, which == 0 ? kMomentum : kRms, tr[p].shape, flat.data() + off[p]);
    }
}

CheckpointInfo load_checkpoint(const std::string& path, Model& model, Adam* adam) {
    std::vector<unsigned char> d;
    {
        File file(path, "rb");
        std::fseek(file.f, 0, SEEK_END);
        long sz = std::ftell(file.f);
        std::fseek(file.f, 0, SEEK_SET);
        d.resize(sz > 0 ? (size_t)sz : 0);
        if (!d.empty() && std::fread(d.data(), 1, d.size(), file.f) != d.size())
            throw Error(MTL_ERR_INVALID, "cannot read checkpoint file " + path);
    }
    size_t off = 0;
    if (get_u32(d, off) != kMagic) throw Error(MTL_ERR_INVALID, "Not a mantle checkpoint file (bad magic): " + path);
    const uint32_t version = get_u32(d, off);
    if (version != kVersion) throw Error(MTL_ERR_INVALID, "Unsupported checkpoint version: " + std::to_string(version));
    CheckpointInfo info;
    info.iter = (int)get_u32(d, off);
    const uint32_t n_tensors = get_u32(d, off), n_optim = get_u32(d, off);
    info.has_optim_state = n_optim > 0;

    const std::vector<Symbol>& tr = model.trainable_parameters();
    const std::vector<int64_t>& toff = model.trainable_offsets();
    std::vector<float> m, v;
    if (adam) {
        m.resize((size_t)std::max<int64_t>(model.n_trainable(), 1));
        v.resize(m.size());
        adam->get_state(0, m.data());
        adam->get_state(1, v.data());
    }
    std::vector<float> host;
    for (uint32_t e = 0; e < n_tensors + n_optim; ++e) {
        // _read_entry_header, checkpoint.mojo:119-147
        const uint32_t id = get_u32(d, off);
        if (off + 1 > d.size()) throw Error(MTL_ERR_INVALID, "checkpoint file is truncated");
        const uint8_t kind = d[off++];
        const uint32_t rank = get_u32(d, off);
        if (rank > (uint32_t)MTL_MAX_RANK) throw Error(MTL_ERR_INVALID, "checkpoint entry has rank above 8");
        // Dimensions are untrusted: bound every partial product by the floats the rest of the file can
        // still hold, so that neither the element count nor the byte count can wrap around.
        uint64_t n = 1;
        for (uint32_t i = 0; i < rank; ++i) {
            const uint64_t dim = get_u32(d, off);
            const uint64_t room = (uint64_t)(d.size() - std::min(off, d.size())) / 4;
            if (dim != 0 && n > room / dim)
                throw Error(MTL_ERR_INVALID, "checkpoint entry for symbol " + std::to_string(id) +
                                                 " declares more elements than the file holds");
            n *= dim;
        }
        const size_t bytes = (size_t)n * 4;
        if (off > d.size() || bytes > d.size() - off) throw Error(MTL_ERR_INVALID, "checkpoint file is truncated");
        host.resize((size_t)n);
        std::memcpy(host.data(), d.data() + off, bytes);
        off += bytes;
        if (e < n_tensors) {
            if (!model.has_tensor((int)id)) continue;  // unknown symbol: skipped, as the reference does
            if ((uint64_t)model.shape_of((int)id).num_elements() != n)
                throw Error(MTL_ERR_INVALID, "checkpoint entry for symbol " + std::to_string(id) + " has another size");
            model.set_tensor((int)id, host.data());
        } else if (adam) {
            for (size_t p = 0; p < tr.size(); ++p) {
                if ((uint32_t)tr[p].id != id) continue;
                if ((uint64_t)tr[p].shape.num_elements() != n)
                    throw Error(MTL_ERR_INVALID, "optimizer entry for symbol " + std::to_string(id) + " has another size");
                float* dst = (kind == kMomentum ? m.data() : v.data()) + toff[p];
                std::memcpy(dst, host.data(), bytes);
            }
        }
    }
    if (adam && info.has_optim_state) {
        adam->set_state(0, m.data());
        adam->set_state(1, v.data());
        adam->set_iter(info.iter);
    }
    return info;
}

}  // namespace mantle
