// Native checkpoint files (mantle/serialize/checkpoint.mojo:22-470): "BSLT" version 1.
//   header   u32 magic 0x42534C54 | u32 version 1 | u32 iter | u32 n_tensors | u32 n_optim
//   entry    u32 symbol id | u8 kind (0 tensor, 1 Adam momentum, 2 Adam rms) | u32 rank |
//            u32 dims[rank] | fp32 data, row-major, little endian
// Tensors are every entry of Parameters.tensors in allocation order (inputs, parameters, node
// outputs); optimizer entries are all momentum tensors, then all rms tensors, in
// get_trainable_parameters order.  Loading matches entries by symbol id and skips ids the model
// does not have (checkpoint.mojo:150-167).  Data moves between the file and the device arenas.
#pragma once

#include <string>

#include "model.hpp"

namespace mantle {

struct CheckpointInfo {
    int iter = 0;
    bool has_optim_state = false;
};

// adam == nullptr: save_checkpoint (no optimizer entries); else save_checkpoint_with_optim.
void save_checkpoint(const std::string& path, const Model& model, const Adam* adam, int iter);
// adam == nullptr: load_checkpoint (optimizer entries are skipped); else load_checkpoint_with_optim,
// which also sets the optimizer's step count to the stored one.
CheckpointInfo load_checkpoint(const std::string& path, Model& model, Adam* adam);

}  // namespace mantle
