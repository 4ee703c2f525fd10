// Tensor<dtype, device> and MemoryBuffer<device> with the field and method names of anyGPU's
// srcs/core/tensor.hpp:19-128 (MemoryBuffer) and :147-247 (Tensor): id, dim, offset (bytes), alignment, shape, stride
// (elements), name; buffer(), raw_buffer(), numel(), size(), capacity(), copy_to_host(), copy_to_cuda().
// Like anyGPU's, device buffers are zero-filled on allocation (srcs/core/tensor.hpp:80-84); host buffers come from
// std::aligned_alloc and are zero-filled too.
#pragma once

#include <memory>
#include <random>

#include "core.hpp"

template <Device device>
struct MemoryBuffer
{
	int64 id;
	int64 capacity;  // bytes
	char* buffer;

	explicit MemoryBuffer(const int64 capacity_bytes) : id(GlobalUUIDGenerator::generate_id()), capacity(capacity_bytes), buffer(nullptr)
	{
		if (capacity == 0) return;
		if constexpr (device == CPU)
		{
			const size_t rounded = (static_cast<size_t>(capacity) + 255u) & ~static_cast<size_t>(255u);
			buffer = static_cast<char*>(std::aligned_alloc(256, rounded));
			std::memset(buffer, 0, rounded);
		}
		else
		{
			CUDA_CHECK(cudaMalloc(&buffer, static_cast<size_t>(capacity)));
			CUDA_CHECK(cudaMemset(buffer, 0, static_cast<size_t>(capacity)));  // as anyGPU does: code written against it may rely on zeros
		}
	}
	MemoryBuffer(const MemoryBuffer&) = delete;
	MemoryBuffer& operator=(const MemoryBuffer&) = delete;
	~MemoryBuffer()
	{
		if (!buffer) return;
		if constexpr (device == CPU) std::free(buffer);
		else cudaFree(buffer);
	}
};

template <typename dtype, Device device = CUDA>
struct Tensor
{
	int64 id;
	int64 dim;
	int64 offset;     // bytes into the buffer
	int64 alignment;  // bytes
	Shape shape;
	Stride stride;    // elements
	std::string name;

	dtype* buffer() const { return reinterpret_cast<dtype*>(mem_buffer->buffer + offset); }
	char* raw_buffer() const { return mem_buffer->buffer; }
	int64 numel() const { return calc_default_size(dim, shape); }
	int64 size() const { return dim == 0 ? 0 : shape[0] * stride[0]; }
	int64 capacity() const { return mem_buffer->capacity; }
	int64 buffer_id() const { return mem_buffer->id; }

	Tensor() : id(GlobalUUIDGenerator::generate_id()), dim(0), offset(0), alignment(1), shape{}, stride{} {}

	explicit Tensor(const int64 capacity_bytes) : Tensor()
	{
		mem_buffer = std::make_shared<MemoryBuffer<device>>(capacity_bytes);
	}

	explicit Tensor(const std::vector<int64>& shp) : Tensor()
	{
		dim = static_cast<int64>(shp.size());
		shape = cvt_vector2array(shp);
		stride = calc_default_stride(dim, shape);
		mem_buffer = std::make_shared<MemoryBuffer<device>>(static_cast<int64>(sizeof(dtype)) * calc_default_size(shp));
	}

	explicit Tensor(const int64 d, const Shape& shp) : Tensor()
	{
		dim = d;
		shape = shp;
		stride = calc_default_stride(dim, shape);
		mem_buffer = std::make_shared<MemoryBuffer<device>>(static_cast<int64>(sizeof(dtype)) * calc_default_size(dim, shape));
	}

	explicit Tensor(const std::vector<int64>& shp, const std::vector<dtype>& hdata) : Tensor(shp)
	{
		const size_t bytes = sizeof(dtype) * hdata.size();
		if constexpr (device == CPU) std::memcpy(mem_buffer->buffer, hdata.data(), bytes);
		else CUDA_CHECK(cudaMemcpy(mem_buffer->buffer, hdata.data(), bytes, cudaMemcpyHostToDevice));
	}

	Tensor<dtype, CPU> copy_to_host() const { return copy_to<CPU>(); }
	Tensor<dtype, CUDA> copy_to_cuda() const { return copy_to<CUDA>(); }

	// Shares the buffer of `other` (used by the view / slice helpers).
	template <typename T2, Device D2> friend struct Tensor;
	std::shared_ptr<MemoryBuffer<device>> mem_buffer;

private:
	template <Device target>
	Tensor<dtype, target> copy_to() const
	{
		Tensor<dtype, target> t(mem_buffer->capacity);
		t.dim = dim;
		t.shape = shape;
		t.stride = stride;
		t.alignment = alignment;
		t.offset = offset;
		t.name = name;
		if (mem_buffer->capacity == 0) return t;
		cudaMemcpyKind kind = cudaMemcpyHostToHost;
		if (device == CPU && target == CUDA) kind = cudaMemcpyHostToDevice;
		if (device == CUDA && target == CPU) kind = cudaMemcpyDeviceToHost;
		if (device == CUDA && target == CUDA) kind = cudaMemcpyDeviceToDevice;
		if (kind == cudaMemcpyHostToHost) std::memcpy(t.mem_buffer->buffer, mem_buffer->buffer, static_cast<size_t>(mem_buffer->capacity));
		else CUDA_CHECK(cudaMemcpy(t.mem_buffer->buffer, mem_buffer->buffer, static_cast<size_t>(mem_buffer->capacity), kind));
		return t;
	}
};

// tensor_view (anyGPU srcs/ops/shape_ops.hpp:10-20): same buffer, new shape, default strides.
template <typename dtype, Device device>
inline Tensor<dtype, device> tensor_view(const Tensor<dtype, device>& x, const std::vector<int64>& new_shape)
{
	Tensor<dtype, device> y = x;
	y.id = GlobalUUIDGenerator::generate_id();
	y.dim = static_cast<int64>(new_shape.size());
	y.shape = cvt_vector2array(new_shape);
	y.stride = calc_default_stride(y.dim, y.shape);
	y.name = "";
	return y;
}

// Last-axis slice WITHOUT a copy: same buffer, byte offset advanced, row stride kept. (anyGPU's tensor_slice copies row by
// row, srcs/ops/shape_ops.hpp:190-254; the kernels of this library take row strides, so the view is enough.)
template <typename dtype, Device device>
inline Tensor<dtype, device> tensor_slice_view(const Tensor<dtype, device>& x, const int64 lo, const int64 hi)
{
	Tensor<dtype, device> y = x;
	y.id = GlobalUUIDGenerator::generate_id();
	y.shape[x.dim - 1] = hi - lo;
	y.offset = x.offset + lo * static_cast<int64>(sizeof(dtype));
	y.name = "";
	return y;
}

// tensor_slice(x, axis, lo, hi) of anyGPU (srcs/ops/shape_ops.hpp:190-254): a NEW contiguous tensor holding x[..., lo:hi, ...]
// along `axis`. anyGPU issues one cudaMemcpy per outer row from a host loop; here the tensor is seen as [outer, shape[axis], inner]
// and one 2-D copy moves `outer` rows of (hi - lo) * inner elements. x must be contiguous (default strides), as in anyGPU.
template <typename dtype, Device device>
inline Tensor<dtype, device> tensor_slice(const Tensor<dtype, device>& x, const int64 axis, const int64 lo, const int64 hi)
{
	ACASSERT(axis >= 0 && axis < x.dim, "tensor_slice: axis out of range");
	ACASSERT(0 <= lo && lo <= hi && hi <= x.shape[axis], "tensor_slice: bounds out of range");
	Tensor<dtype, device> y(x.dim, [&] { Shape s = x.shape; s[axis] = hi - lo; return s; }());
	int64 outer = 1, inner = 1;
	for (int64 i = 0; i < axis; ++i) outer *= x.shape[i];
	for (int64 i = axis + 1; i < x.dim; ++i) inner *= x.shape[i];
	const size_t width = static_cast<size_t>((hi - lo) * inner) * sizeof(dtype);
	const size_t src_pitch = static_cast<size_t>(x.shape[axis] * inner) * sizeof(dtype);
	if (width == 0 || outer == 0) return y;
	const char* src = reinterpret_cast<const char*>(x.buffer()) + static_cast<size_t>(lo * inner) * sizeof(dtype);
	if constexpr (device == CPU)
	{
		for (int64 r = 0; r < outer; ++r) std::memcpy(reinterpret_cast<char*>(y.buffer()) + r * width, src + r * src_pitch, width);
	}
	else
	{
		CUDA_CHECK(cudaMemcpy2DAsync(y.buffer(), width, src, src_pitch, width, static_cast<size_t>(outer), cudaMemcpyDeviceToDevice, 0));
	}
	return y;
}

// Seeded creators (anyGPU srcs/core/tensor.hpp:490-506, :533-547).
template <typename dtype, Device device>
inline Tensor<dtype, device> crt_random_normal_tensor(const std::vector<int64>& shape, const int64 seed = 10, const float scale = 1.0f)
{
	std::default_random_engine eng(static_cast<unsigned>(seed));
	std::normal_distribution<float32> dist(0.f, 1.f);
	std::vector<dtype> h(static_cast<size_t>(calc_default_size(shape)));
	for (auto& v : h) v = static_cast<dtype>(dist(eng) * scale);
	return Tensor<dtype, device>(shape, h);
}

template <typename dtype, Device device>
inline Tensor<dtype, device> crt_ones_tensor(const std::vector<int64>& shape)
{
	std::vector<dtype> h(static_cast<size_t>(calc_default_size(shape)), static_cast<dtype>(1.0f));
	return Tensor<dtype, device>(shape, h);
}

// f16 <-> f32 conversion of host tensors (anyGPU converts to float32 only, srcs/core/tensor.hpp:388-410).
template <typename trg, typename src>
inline Tensor<trg, CPU> cvt_tensor_datatype(const Tensor<src, CPU>& t)
{
	Tensor<trg, CPU> out(t.dim, t.shape);
	const int64 n = t.numel();
	for (int64 i = 0; i < n; ++i)
	{
		float v;
		if constexpr (std::is_same_v<src, float16>) v = __half2float(t.buffer()[i]);
		else v = static_cast<float>(t.buffer()[i]);
		if constexpr (std::is_same_v<trg, float16>) out.buffer()[i] = __float2half_rn(v);
		else out.buffer()[i] = static_cast<trg>(v);
	}
	return out;
}
