#include "runtime/Generator.h"

#include <ATen/Utils.h>
#include <ATen/EmptyTensor.h>

#include <cstring>
#include <deque>
#include <mutex>
#include <vector>

namespace supa {

SupaGeneratorImpl::SupaGeneratorImpl(c10::DeviceIndex device_index)
    : c10::GeneratorImpl{c10::Device(c10::DeviceType::PrivateUse1, device_index),
                         c10::DispatchKeySet(c10::DispatchKey::PrivateUse1)} {}

void SupaGeneratorImpl::set_current_seed(uint64_t seed) {
  seed_ = seed;
  offset_ = 0;
}

void SupaGeneratorImpl::set_offset(uint64_t offset) {
  TORCH_CHECK(offset % 4 == 0, "offset must be a multiple of 4");
  offset_ = offset;
}

uint64_t SupaGeneratorImpl::get_offset() const { return offset_; }
uint64_t SupaGeneratorImpl::current_seed() const { return seed_; }

uint64_t SupaGeneratorImpl::seed() {
  const uint64_t random = c10::detail::getNonDeterministicRandom(true);
  set_current_seed(random);
  return random;
}

namespace {
constexpr size_t kSeedBytes = sizeof(uint64_t);
constexpr size_t kStateBytes = kSeedBytes + sizeof(int64_t);
}  // namespace

c10::intrusive_ptr<c10::TensorImpl> SupaGeneratorImpl::get_state() const {
  auto state = at::detail::empty_cpu({static_cast<int64_t>(kStateBytes)}, at::ScalarType::Byte, c10::nullopt, c10::nullopt,
                                     c10::nullopt, c10::nullopt);
  uint8_t* raw = state.data_ptr<uint8_t>();
  const int64_t offset = static_cast<int64_t>(offset_);
  std::memcpy(raw, &seed_, kSeedBytes);
  std::memcpy(raw + kSeedBytes, &offset, sizeof(offset));
  return state.getIntrusivePtr();
}

void SupaGeneratorImpl::set_state(const c10::TensorImpl& new_state) {
  at::detail::check_rng_state(new_state);
  const int64_t n = new_state.numel();
  TORCH_CHECK(n == static_cast<int64_t>(kStateBytes) || n == static_cast<int64_t>(kSeedBytes), "RNG state is wrong size");
  const uint8_t* raw = new_state.data_dtype_initialized<uint8_t>();
  uint64_t seed = 0;
  int64_t offset = 0;
  std::memcpy(&seed, raw, kSeedBytes);
  if (n == static_cast<int64_t>(kStateBytes)) std::memcpy(&offset, raw + kSeedBytes, sizeof(offset));
  set_current_seed(seed);
  set_offset(static_cast<uint64_t>(offset));
}

std::pair<uint64_t, uint64_t> SupaGeneratorImpl::philox_engine_inputs(uint64_t increment) {
  const uint64_t offset = offset_;
  offset_ += ((increment + 3) / 4) * 4;
  return {seed_, offset};
}

SupaGeneratorImpl* SupaGeneratorImpl::clone_impl() const {
  auto* gen = new SupaGeneratorImpl(device().index());
  gen->seed_ = seed_;
  gen->offset_ = offset_;
  return gen;
}

namespace {
std::once_flag g_init;
std::deque<std::once_flag> g_gen_once;
std::vector<at::Generator> g_default;

c10::DeviceIndex resolve(c10::DeviceIndex idx) {
  const c10::DeviceIndex n = device_count();
  if (idx == -1) idx = current_device();
  TORCH_CHECK(idx >= 0 && idx < n, "The device_index is invalid.");
  return idx;
}
}  // namespace

const at::Generator& default_generator(c10::DeviceIndex device_index) {
  std::call_once(g_init, [] {
    const c10::DeviceIndex n = device_count();
    g_gen_once.resize(n);
    g_default.resize(n);
  });
  const c10::DeviceIndex idx = resolve(device_index);
  std::call_once(g_gen_once[idx], [&] { g_default[idx] = at::make_generator<SupaGeneratorImpl>(idx); });
  return g_default[idx];
}

at::Generator new_generator(c10::DeviceIndex device_index) {
  return at::make_generator<SupaGeneratorImpl>(resolve(device_index));
}

SupaGeneratorImpl* generator_or_default(const c10::optional<at::Generator>& gen, c10::DeviceIndex device_index) {
  if (gen.has_value() && gen->defined()) {
    TORCH_CHECK(gen->device().type() == c10::DeviceType::PrivateUse1, "Expected a 'supa' device type for generator but found '",
                gen->device().type(), "'");
    return at::check_generator<SupaGeneratorImpl>(*gen);
  }
  return at::check_generator<SupaGeneratorImpl>(default_generator(device_index));
}

}  // namespace supa
