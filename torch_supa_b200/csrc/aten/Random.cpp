// Random fills and dropout on the supa device, driven by the device generator's (seed, offset) pair
// (philox_engine_inputs, torch_supa/csrc/aten/SUPAGeneratorImpl.cpp:450-455).  Every operator takes the pair under the
// generator's mutex, advances the offset by one 128-bit block (4) and launches one kernel on the current stream; the value
// of element i depends on (seed, offset, i) alone, so a restored generator state reproduces a tensor bit for bit
// (what test/test_checkpoint_rng.py:12-46 relies on).
#include <torch/library.h>

#include <cmath>
#include <limits>

#include "aten/Common.h"
#include "runtime/Generator.h"

namespace supa {
namespace {

std::pair<uint64_t, uint64_t> next_inputs(const c10::optional<at::Generator>& gen, const at::Tensor& self) {
  SupaGeneratorImpl* g = generator_or_default(gen, self.device().index());
  std::lock_guard<std::mutex> lock(g->mutex_);
  return g->philox_engine_inputs(4);
}

// Fills `self` (any strides: a non-contiguous tensor is filled through a contiguous temporary).
void fill_random(at::Tensor& self, int kind, double a, double b, int64_t low, uint64_t range, const c10::optional<at::Generator>& gen) {
  check_same_device("random fill", {self});
  if (self.numel() == 0) return;
  c10::DeviceGuard guard(self.device());
  const auto inputs = next_inputs(gen, self);
  at::Tensor dst = self.is_contiguous() ? self : at::empty(self.sizes(), self.options());
  sb_rng_args args{};
  args.dst = dst.data_ptr();
  args.dtype = dtype_code(dst.scalar_type());
  args.kind = kind;
  args.numel = dst.numel();
  args.a = a;
  args.b = b;
  args.low = low;
  args.range = range;
  args.seed = inputs.first;
  args.offset = inputs.second;
  check_kernel(sb_rng_fill(&args, stream_of(dst)), "sb_rng_fill");
  if (!dst.is_same(self)) self.copy_(dst);
}

void check_real(const at::Tensor& self, const char* op) {
  TORCH_CHECK_NOT_IMPLEMENTED(at::isFloatingType(self.scalar_type()) && self.scalar_type() != at::kFloat8_e4m3fn &&
                                  self.scalar_type() != at::kFloat8_e5m2,
                              op, ": supa backend supports float, double, half and bfloat16, got ", self.scalar_type());
}

double type_max(at::ScalarType t) {
  switch (t) {
    case at::kHalf: return 65504.0;
    case at::kBFloat16: return 3.3895313892515355e38;
    case at::kFloat: return std::numeric_limits<float>::max();
    default: return std::numeric_limits<double>::max();
  }
}

at::Tensor& uniform_(at::Tensor& self, double from, double to, c10::optional<at::Generator> gen) {
  check_real(self, "uniform_");
  const double top = type_max(self.scalar_type());
  TORCH_CHECK(from >= -top && from <= top, "from is out of bounds for ", self.scalar_type());
  TORCH_CHECK(to >= -top && to <= top, "to is out of bounds for ", self.scalar_type());
  TORCH_CHECK(from <= to, "uniform_ expects to return a [from, to) range, but found from=", from, " > to=", to);
  TORCH_CHECK((to - from) <= std::numeric_limits<double>::max(), "uniform_ expects to-from <= std::numeric_limits<double>::max(), but found to=",
              to, " and from=", from, " which result in to-from to exceed the limit");
  fill_random(self, SB_RNG_UNIFORM, from, to, 0, 0, gen);
  return self;
}

at::Tensor& normal_(at::Tensor& self, double mean, double std, c10::optional<at::Generator> gen) {
  check_real(self, "normal_");
  TORCH_CHECK(std >= 0.0, "normal expects std >= 0.0, but found std ", std);
  fill_random(self, SB_RNG_NORMAL, mean, std, 0, 0, gen);
  return self;
}

// Largest value random_() may return for the dtype: 2^mantissa for floating types (every integer up to it is representable),
// the type's maximum for integers.
int64_t random_upper_inclusive(at::ScalarType t) {
  switch (t) {
    case at::kBool: return 1;
    case at::kByte: return std::numeric_limits<uint8_t>::max();
    case at::kChar: return std::numeric_limits<int8_t>::max();
    case at::kShort: return std::numeric_limits<int16_t>::max();
    case at::kInt: return std::numeric_limits<int32_t>::max();
    case at::kLong: return std::numeric_limits<int64_t>::max();
    case at::kHalf: return int64_t(1) << 11;
    case at::kBFloat16: return int64_t(1) << 8;
    case at::kFloat: return int64_t(1) << 24;
    case at::kDouble: return int64_t(1) << 53;
    default: TORCH_CHECK_NOT_IMPLEMENTED(false, "random_: supa backend does not support ", t);
  }
}

at::Tensor& random_from_to(at::Tensor& self, int64_t from, c10::optional<int64_t> to, c10::optional<at::Generator> gen) {
  const at::ScalarType t = self.scalar_type();
  const int64_t top = random_upper_inclusive(t);
  uint64_t range;
  if (to.has_value()) {
    TORCH_CHECK(from < *to, "random_ expects 'from' to be less than 'to', but got from=", from, " >= to=", *to);
    if (at::isFloatingType(t)) {
      TORCH_CHECK(from >= -top && *to - 1 <= top, "random_: from=", from, " to=", *to, " is out of the range ", t, " represents exactly");
    } else if (t != at::kLong) {
      const int64_t low = t == at::kBool || t == at::kByte ? 0 : -top - 1;
      TORCH_CHECK(from >= low && *to - 1 <= top, "random_: from=", from, " to=", *to, " is out of bounds for ", t);
    }
    range = static_cast<uint64_t>(*to) - static_cast<uint64_t>(from);
  } else {
    // [from, top]; the whole 64-bit range is written as 0
    range = static_cast<uint64_t>(top) - static_cast<uint64_t>(from) + 1;
  }
  fill_random(self, SB_RNG_INTEGER, 0, 0, from, range, gen);
  return self;
}

at::Tensor& random_to(at::Tensor& self, int64_t to, c10::optional<at::Generator> gen) { return random_from_to(self, 0, to, gen); }

at::Tensor& random_(at::Tensor& self, c10::optional<at::Generator> gen) {
  const int64_t top = random_upper_inclusive(self.scalar_type());
  fill_random(self, SB_RNG_INTEGER, 0, 0, 0, static_cast<uint64_t>(top) + 1, gen);
  return self;
}

at::Tensor& bernoulli_float(at::Tensor& self, double p, c10::optional<at::Generator> gen) {
  TORCH_CHECK(0 <= p && p <= 1, "bernoulli_ expects p to be in [0, 1], but got p=", p);
  fill_random(self, SB_RNG_BERNOULLI, p, 0, 0, 0, gen);
  return self;
}

// out = input * mask / (1 - p), mask ~ Bernoulli(1 - p); one kernel reads the input and writes both.
std::tuple<at::Tensor, at::Tensor> native_dropout(const at::Tensor& input, double p, c10::optional<bool> train) {
  check_same_device("native_dropout", {input});
  TORCH_CHECK(p >= 0 && p <= 1, "dropout probability has to be between 0 and 1, but got ", p);
  c10::DeviceGuard guard(input.device());
  const at::ScalarType t = input.scalar_type();
  if (input.numel() == 0) return {at::empty_like(input), at::empty_like(input, input.options().dtype(at::kBool))};
  if ((train.has_value() && !*train) || p == 0.0) {
    return {input.clone(), at::ones_like(input, input.options().dtype(at::kBool), at::MemoryFormat::Contiguous)};
  }
  TORCH_CHECK_NOT_IMPLEMENTED(t == at::kFloat || t == at::kHalf || t == at::kBFloat16, "native_dropout: supa backend supports float, half and bfloat16, got ", t);
  const at::Tensor x = input.contiguous();
  at::Tensor out = at::empty_like(x, at::MemoryFormat::Contiguous);
  at::Tensor mask = at::empty(x.sizes(), x.options().dtype(at::kBool));
  const auto inputs = next_inputs(c10::nullopt, x);
  check_kernel(sb_dropout(x.data_ptr(), out.data_ptr(), mask.data_ptr(), dtype_code(t), x.numel(), p, inputs.first, inputs.second, stream_of(x)),
               "sb_dropout");
  return {out, mask};
}

at::Tensor native_dropout_backward(const at::Tensor& grad_output, const at::Tensor& mask, double scale) {
  check_same_device("native_dropout_backward", {grad_output, mask});
  return (grad_output * mask.to(grad_output.scalar_type())) * scale;
}

}  // namespace
}  // namespace supa

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("uniform_", TORCH_FN(supa::uniform_));
  m.impl("normal_", TORCH_FN(supa::normal_));
  m.impl("random_.from", TORCH_FN(supa::random_from_to));
  m.impl("random_.to", TORCH_FN(supa::random_to));
  m.impl("random_", TORCH_FN(supa::random_));
  m.impl("bernoulli_.float", TORCH_FN(supa::bernoulli_float));
  m.impl("native_dropout", TORCH_FN(supa::native_dropout));
  m.impl("native_dropout_backward", TORCH_FN(supa::native_dropout_backward));
}
