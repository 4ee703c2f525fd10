// Reads a .safetensors file with include/anygpu/io/safetensors_file.hpp (host code only: no device is touched) and prints,
// per tensor, name, stored type, shape and the float64 sum and sum of squares of its float32 conversion; the Python test that
// wrote the file compares them with its own numbers.
#include <cstdio>

#include "anygpu/io/safetensors_file.hpp"

int main(int argc, char** argv)
{
	if (argc < 2) return 2;
	const std::string path = argv[1];
	for (const auto& info : sft_read_tensorinfos(path))
	{
		const auto t = sft_read_tensor_f32(path, info.name);
		double s = 0.0, s2 = 0.0;
		for (int64 i = 0; i < t.numel(); ++i)
		{
			s += t.buffer()[i];
			s2 += static_cast<double>(t.buffer()[i]) * t.buffer()[i];
		}
		std::printf("%s %s", info.name.c_str(), info.dtype.c_str());
		for (auto d : info.shape) std::printf(" %lld", static_cast<long long>(d));
		std::printf(" | %.9e %.9e\n", s, s2);
	}
	return 0;
}
