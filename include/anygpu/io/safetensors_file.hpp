// Reader of .safetensors checkpoints for the tensors of a Mamba2 mixer: 8-byte little-endian header length, a JSON header
// {"name": {"dtype": "F32|F16|BF16", "shape": [...], "data_offsets": [begin, end]}, ..., "__metadata__": {...}}, then the
// raw tensor bytes (offsets relative to the end of the header). Same job and entry-point names as anyGPU's reader
// (srcs/io/safetensors_file.hpp:7-100, srcs/io/safetensors_file.cpp:77-128); additionally one tensor can be fetched by name
// and converted to float32 whatever it is stored as (Zamba2 checkpoints are BF16, which anyGPU's typed reader rejects).
#pragma once

#include <cctype>
#include <cstring>
#include <fstream>
#include <unordered_map>

#include "../tensor.hpp"

struct TensorInfo
{
	unsigned long long offset_start = 0;  // relative to the first byte after the header
	unsigned long long offset_end = 0;
	std::vector<int64> shape;
	std::string dtype;  // "F32", "F16", "BF16", ...
	std::string name;
};

namespace sft_detail {
// Minimal JSON walk: strings, integers, arrays of integers and nested objects are all the format uses.
struct Cursor
{
	const std::string& s;
	size_t i = 0;
	void skip_ws() { while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i; }
	bool eat(char c) { skip_ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return false; }
	char peek() { skip_ws(); return i < s.size() ? s[i] : '\0'; }
	std::string str()
	{
		std::string out;
		if (!eat('"')) return out;
		while (i < s.size() && s[i] != '"')
		{
			if (s[i] == '\\' && i + 1 < s.size()) ++i;  // keep the escaped character as it is
			out.push_back(s[i++]);
		}
		++i;
		return out;
	}
	std::vector<int64> int_list()
	{
		std::vector<int64> v;
		if (!eat('[')) return v;
		while (peek() != ']' && i < s.size())
		{
			skip_ws();
			int64 n = 0;
			while (i < s.size() && std::isdigit(static_cast<unsigned char>(s[i]))) n = n * 10 + (s[i++] - '0');
			v.push_back(n);
			eat(',');
		}
		eat(']');
		return v;
	}
	// skips any value (used for __metadata__ and unknown keys)
	void skip_value()
	{
		const char c = peek();
		if (c == '"') { str(); return; }
		if (c == '{' || c == '[')
		{
			const char open = c, close = c == '{' ? '}' : ']';
			int depth = 0;
			do
			{
				if (s[i] == '"') { str(); continue; }
				if (s[i] == open) ++depth;
				if (s[i] == close) --depth;
				++i;
			} while (depth > 0 && i < s.size());
			return;
		}
		while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']') ++i;
	}
};

inline float bf16_to_f32(uint16_t b)
{
	const uint32_t u = static_cast<uint32_t>(b) << 16;
	float f;
	std::memcpy(&f, &u, sizeof(f));
	return f;
}
}  // namespace sft_detail

// Tensor infos of a JSON header string, in file order.
inline void _sft_read_tensorinfo_from_json(const std::string& header_content, std::vector<TensorInfo>& tensor_infos)
{
	sft_detail::Cursor c{ header_content };
	if (!c.eat('{')) return;
	while (c.peek() == '"')
	{
		const std::string name = c.str();
		c.eat(':');
		if (name == "__metadata__" || c.peek() != '{')
		{
			c.skip_value();
		}
		else
		{
			TensorInfo info;
			info.name = name;
			c.eat('{');
			while (c.peek() == '"')
			{
				const std::string key = c.str();
				c.eat(':');
				if (key == "dtype") info.dtype = c.str();
				else if (key == "shape") info.shape = c.int_list();
				else if (key == "data_offsets")
				{
					const auto o = c.int_list();
					ACASSERT(o.size() == 2, "exactly two offset values are needed");
					info.offset_start = static_cast<unsigned long long>(o[0]);
					info.offset_end = static_cast<unsigned long long>(o[1]);
				}
				else c.skip_value();
				c.eat(',');
			}
			c.eat('}');
			tensor_infos.push_back(info);
		}
		c.eat(',');
	}
}

// Header of a file: tensor infos and the position of the first data byte.
inline std::vector<TensorInfo> sft_read_tensorinfos(const std::string& path, unsigned long long* data_begin = nullptr)
{
	std::ifstream f(path, std::ios::binary);
	if (!f.is_open())
	{
		log_error("Unable to open file: " + path);
		exit(1);
	}
	f.seekg(0, std::ios::end);
	const unsigned long long file_size = static_cast<unsigned long long>(f.tellg());
	f.seekg(0, std::ios::beg);
	unsigned long long header_size = 0;
	f.read(reinterpret_cast<char*>(&header_size), sizeof(header_size));
	// a truncated or corrupt file must not turn into an unbounded allocation or silently empty tensors
	if (!f || file_size < 8 || header_size > file_size - 8)
	{
		log_error("Not a safetensors file (header length exceeds the file): " + path);
		exit(1);
	}
	std::string header(static_cast<size_t>(header_size), '\0');
	f.read(header.data(), static_cast<std::streamsize>(header_size));
	if (!f)
	{
		log_error("Unable to read the safetensors header: " + path);
		exit(1);
	}
	std::vector<TensorInfo> infos;
	_sft_read_tensorinfo_from_json(header, infos);
	const unsigned long long data_bytes = file_size - 8ull - header_size;
	for (const auto& info : infos)
	{
		if (info.offset_end < info.offset_start || info.offset_end > data_bytes)
		{
			log_error("safetensors data_offsets of '" + info.name + "' lie outside the file: " + path);
			exit(1);
		}
	}
	if (data_begin) *data_begin = 8ull + header_size;
	return infos;
}

// One tensor by name as float32, converted from F32 / F16 / BF16 storage.
inline Tensor<float32, CPU> sft_read_tensor_f32(const std::string& path, const std::string& name)
{
	unsigned long long data_begin = 0;
	const auto infos = sft_read_tensorinfos(path, &data_begin);
	for (const auto& info : infos)
	{
		if (info.name != name) continue;
		Tensor<float32, CPU> t(info.shape);
		const size_t n = static_cast<size_t>(t.numel());
		const size_t bytes = static_cast<size_t>(info.offset_end - info.offset_start);
		std::ifstream f(path, std::ios::binary);
		f.seekg(static_cast<std::streamoff>(data_begin + info.offset_start));
		if (info.dtype == "F32")
		{
			ACASSERT(bytes == n * 4, "data_offsets do not match the shape");
			f.read(reinterpret_cast<char*>(t.buffer()), static_cast<std::streamsize>(bytes));
			ACASSERT(static_cast<bool>(f), "short read of tensor data");
		}
		else if (info.dtype == "F16" || info.dtype == "BF16")
		{
			ACASSERT(bytes == n * 2, "data_offsets do not match the shape");
			std::vector<uint16_t> raw(n);
			f.read(reinterpret_cast<char*>(raw.data()), static_cast<std::streamsize>(bytes));
			ACASSERT(static_cast<bool>(f), "short read of tensor data");
			for (size_t i = 0; i < n; ++i)
			{
				if (info.dtype == "BF16") t.buffer()[i] = sft_detail::bf16_to_f32(raw[i]);
				else
				{
					__half h;
					std::memcpy(&h, &raw[i], 2);
					t.buffer()[i] = __half2float(h);
				}
			}
		}
		else
		{
			log_error("unsupported data type in safetensors: " + info.dtype);
			exit(1);
		}
		t.name = name;
		return t;
	}
	log_error("tensor not found in " + path + ": " + name);
	exit(1);
}

// All tensors of one stored type (anyGPU's sft_read_tensors, srcs/io/safetensors_file.hpp:30-100), here always as float32.
inline void sft_read_tensors(const std::string& path, std::unordered_map<std::string, Tensor<float32, CPU>>& tensors)
{
	for (const auto& info : sft_read_tensorinfos(path)) tensors.emplace(info.name, sft_read_tensor_f32(path, info.name));
}
