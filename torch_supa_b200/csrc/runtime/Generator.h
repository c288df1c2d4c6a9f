// Random number generator of the supa device: a 64-bit seed and a Philox offset, handed to kernels as a pair.  Counterpart of
// SUPAGeneratorImpl (torch_supa/csrc/aten/SUPAGeneratorImpl.cpp:196-520) without the graph-capture state, which this
// backend does not have.
#pragma once

#include <ATen/core/Generator.h>
#include <c10/core/GeneratorImpl.h>

#include <utility>

#include "runtime/Runtime.h"

namespace supa {

class SUPA_EXPORT SupaGeneratorImpl final : public c10::GeneratorImpl {
 public:
  explicit SupaGeneratorImpl(c10::DeviceIndex device_index);
  ~SupaGeneratorImpl() override = default;

  // Sets the seed and rewinds the offset to 0.
  void set_current_seed(uint64_t seed) override;
  // The offset counts 32-bit words per stream lane and must stay a multiple of 4 (one 128-bit Philox block).
  void set_offset(uint64_t offset) override;
  uint64_t get_offset() const override;
  uint64_t current_seed() const override;
  // Seeds from a non-deterministic source and returns the seed.
  uint64_t seed() override;
  // The state is 16 bytes, seed then offset (little endian), as a CPU byte tensor; set_state also accepts the 8-byte form
  // that holds the seed alone.
  void set_state(const c10::TensorImpl& new_state) override;
  c10::intrusive_ptr<c10::TensorImpl> get_state() const override;

  // Returns {seed, offset} for a kernel that consumes `increment` words per lane and advances the offset by the increment
  // rounded up to a multiple of 4.  Call with mutex_ held.
  std::pair<uint64_t, uint64_t> philox_engine_inputs(uint64_t increment);

  static c10::DeviceType device_type() { return c10::DeviceType::PrivateUse1; }

 private:
  SupaGeneratorImpl* clone_impl() const override;
  uint64_t seed_ = c10::default_rng_seed_val;
  uint64_t offset_ = 0;
};

// The per-device default generator (created on first use, seeded with the default seed).
const at::Generator& default_generator(c10::DeviceIndex device_index = -1);
// A fresh generator with the default seed.
at::Generator new_generator(c10::DeviceIndex device_index = -1);
// `gen` when it is defined (it must be a supa generator), else the default generator of `device_index`.
SupaGeneratorImpl* generator_or_default(const c10::optional<at::Generator>& gen, c10::DeviceIndex device_index);

}  // namespace supa
