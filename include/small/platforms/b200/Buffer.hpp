// Buffer.hpp -- FloatBuffer / QUInt8Buffer of the B200 platform.
//
// Same public surface as the reference's CPU buffers (platforms/reference/FloatBuffer.hpp
// :42-168, QUInt8Buffer.hpp:31-276: value/accum typedefs, blocking constants, deep copy,
// pointer-swapping move and swap, data(), operator[], size(), zero(), and for uint8 the
// public quantisation fields).  Storage is CUDA managed memory obtained through the C ABI,
// so the reference's host-side helpers (pack_buffer, init, file readers) keep working on
// data().  Layer calls are asynchronous; any host access through data() or operator[]
// first waits for outstanding device work, and the next layer call moves a host-touched
// buffer back to the device before launching.
#pragma once

#include <small_b200.h>
#include <stdint.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <new>
#include <stdexcept>
#include <string>
#include <type_traits>

namespace small
{
namespace b200
{
// True while layer calls may still be running on the device.
inline bool &pending()
{
    static bool p = false;
    return p;
}

// Images per call for the batched extension (image-major batch); 1 = the reference.
inline int &batch()
{
    static thread_local int n = 1;
    return n;
}

struct BatchScope
{
    int saved;
    explicit BatchScope(int n) : saved(batch()) { batch() = n; }
    ~BatchScope() { batch() = saved; }
};

// Stride along the height for the layer calls of this thread when it differs from the stride argument
// (0 = the same on both axes).  The 1-D family is the 2-D functions with a window height of 1 and a
// row stride of 1: its wrappers open a RowStrideScope(1) around the 2-D call.
inline int &row_stride()
{
    static thread_local int s = 0;
    return s;
}

struct RowStrideScope
{
    int saved;
    explicit RowStrideScope(int s) : saved(row_stride()) { row_stride() = s; }
    ~RowStrideScope() { row_stride() = saved; }
};

// Stream the layer calls of this thread are enqueued on (nullptr = the default stream), and
// whether that stream is being captured into a graph (see InferenceGraph below).
inline void *&stream()
{
    static thread_local void *s = nullptr;
    return s;
}
inline bool &capturing()
{
    static thread_local bool c = false;
    return c;
}

struct StreamScope
{
    void *saved;
    explicit StreamScope(void *s); // flushes a deferred convolution first: it belongs to the old stream
    ~StreamScope();
};

inline void throw_on(int rc)
{
    if (rc == SMALL_B200_OK)
        return;
    std::string msg(small_b200_last_error());
    if (rc == SMALL_B200_INVALID_ARGUMENT)
        throw std::invalid_argument(msg);
    if (rc == SMALL_B200_OUT_OF_MEMORY)
        throw std::bad_alloc();
    throw std::runtime_error(msg);
}

// A float convolution that has been described but not launched yet.  The reference's layer classes
// run a convolution and its activation as two calls (Conv2DLayer.hpp:827-878: Bias, PartialConv2D,
// then ReLUActivation / LeakyReLUActivation in place); on a GPU the second call is a whole extra
// pass over the activation.  So a convolution call only records itself here, and
//   * an in-place activation of exactly its output, as the next call, becomes the convolution's own
//     epilogue (the bytes in the buffer afterwards are the same: the fused epilogue computes the
//     same function of the same sums);
//   * anything else -- another layer call (every call fetches its buffers with device_ptr()), host
//     access to any buffer, the end of a graph capture, a change of stream, the destruction of a
//     buffer -- launches it first.
// Only calls whose arguments the library accepts are deferred, so argument errors still surface at
// the call that made them.
struct DeferredConv
{
    bool valid = false;
    bool tensor_core = false; // small_b200_conv2d_f32_tf32x3 (filt = the re-laid filter)
    bool depthwise = false;   // small_b200_dwconv2d_f32
    small_b200_layer L{};
    const float *in = nullptr, *filt = nullptr, *bias = nullptr;
    float *out = nullptr;
    void *on_stream = nullptr;
    long long out_elems = 0;
};
inline DeferredConv &deferred()
{
    static thread_local DeferredConv d;
    return d;
}
inline void flush_deferred()
{
    DeferredConv &d = deferred();
    if (!d.valid)
        return;
    d.valid = false;
    throw_on(d.depthwise     ? small_b200_dwconv2d_f32(&d.L, d.in, d.filt, d.bias, d.out, d.on_stream)
             : d.tensor_core ? small_b200_conv2d_f32_tf32x3(&d.L, d.in, d.filt, d.bias, d.out, d.on_stream)
                             : small_b200_conv2d_f32(&d.L, d.in, d.filt, d.bias, d.out, d.on_stream));
}
inline void flush_deferred_quietly() noexcept
{
    try
    {
        flush_deferred();
    }
    catch (...)
    {
    }
}

inline void sync_for_host()
{
    flush_deferred();
    if (capturing())
        throw std::runtime_error("small::b200: host access to a buffer (data(), operator[], copy) while a graph "
                                 "is being captured; a captured inference must only enqueue layer calls");
    if (pending())
    {
        // waits for the device; a kernel that gave up on a bounded wait left stale output behind,
        // which must not reach host code silently: it surfaces here as std::runtime_error
        pending() = false;
        int status = 0;
        throw_on(small_b200_device_status(&status));
    }
}

template <typename T>
class ManagedArray
{
public:
    ManagedArray() : m_num_elts(0), m_buffer(nullptr), m_host_touched(false), m_companion(nullptr), m_companion_key(0) {}

    explicit ManagedArray(size_t num_elts)
        : m_num_elts(num_elts), m_buffer(nullptr), m_host_touched(true), m_companion(nullptr), m_companion_key(0)
    {
        void *p = nullptr;
        if (SMALL_B200_OK != small_b200_malloc_managed(num_elts * sizeof(T), &p))
            throw std::bad_alloc();
        m_buffer = static_cast<T *>(p);
    }

    ManagedArray(ManagedArray const &other) : ManagedArray(other.m_num_elts)
    {
        sync_for_host();
        if (m_num_elts)
            std::memcpy(m_buffer, other.m_buffer, m_num_elts * sizeof(T));
    }

    ManagedArray(ManagedArray &&other) noexcept : ManagedArray() { swap(other); }

    ManagedArray &operator=(ManagedArray const &other)
    {
        if (this != &other)
        {
            ManagedArray tmp(other);
            swap(tmp);
        }
        return *this;
    }

    ManagedArray &operator=(ManagedArray &&other) noexcept
    {
        if (this != &other)
        {
            release();
            swap(other);
        }
        return *this;
    }

    ~ManagedArray() { release(); }

    size_t size() const { return m_num_elts; }

    // Host views: wait for the device, remember that the host may have moved the pages.
    T *data()
    {
        touch();
        return m_buffer;
    }
    T const *data() const
    {
        touch();
        return m_buffer;
    }
    T &operator[](size_t index)
    {
        touch();
        return m_buffer[index];
    }
    T const &operator[](size_t index) const
    {
        touch();
        return m_buffer[index];
    }

    // Element i as the host sees it, without waiting for the device and without marking the buffer
    // host-touched: for small read-only parameters (an activation slope) that no kernel writes.
    T peek(size_t index) const { return m_buffer[index]; }

    void swap(ManagedArray &other) noexcept
    {
        std::swap(m_num_elts, other.m_num_elts);
        std::swap(m_buffer, other.m_buffer);
        std::swap(m_host_touched, other.m_host_touched);
        std::swap(m_companion, other.m_companion);
        std::swap(m_companion_key, other.m_companion_key);
    }

    // A device-only companion derived from the contents (a filter re-laid for the tensor cores).
    // It lives as long as the host does not look at the buffer: data() / operator[] may be
    // followed by writes, so they drop it and the next layer call derives it again.
    T *companion(uint64_t key) const { return (m_companion && m_companion_key == key) ? m_companion : nullptr; }
    T *make_companion(uint64_t key, size_t elems) const
    {
        drop_companion();
        void *p = nullptr;
        if (SMALL_B200_OK != small_b200_malloc(elems * sizeof(T), &p))
            throw std::bad_alloc();
        m_companion = static_cast<T *>(p);
        m_companion_key = key;
        return m_companion;
    }

    // The address without any side effect (to recognise a buffer, never to hand to a kernel).
    T *raw_ptr() const { return m_buffer; }

    // Device view for a layer call: no wait; brings host-touched pages back first.  A convolution that
    // is still waiting for its activation goes first: this call is not that activation.
    T *device_ptr() const
    {
        flush_deferred();
        if (m_host_touched && m_buffer && !capturing()) // a capture only records kernels; pages move on demand
        {
            small_b200_prefetch(m_buffer, m_num_elts * sizeof(T), stream());
            m_host_touched = false;
        }
        pending() = true;
        return m_buffer;
    }

private:
    void touch() const
    {
        if (m_buffer)
        {
            sync_for_host();
            m_host_touched = true;
            drop_companion();
        }
    }

    void drop_companion() const noexcept
    {
        if (m_companion)
        {
            if (pending())
            {
                small_b200_device_sync();
                pending() = false;
            }
            small_b200_free(m_companion);
            m_companion = nullptr;
        }
    }

    void release() noexcept
    {
        if (m_buffer)
        {
            flush_deferred_quietly(); // it may read or write this buffer
            if (pending())
            {
                small_b200_device_sync();
                pending() = false;
            }
            small_b200_free(m_buffer);
        }
        drop_companion();
        m_buffer = nullptr;
        m_num_elts = 0;
    }

    size_t m_num_elts;
    T *m_buffer;
    mutable bool m_host_touched;
    mutable T *m_companion;
    mutable uint64_t m_companion_key;
};
inline StreamScope::StreamScope(void *s) : saved(stream())
{
    flush_deferred();
    stream() = s;
}
inline StreamScope::~StreamScope()
{
    flush_deferred_quietly();
    stream() = saved;
}

// A whole inference as one CUDA graph.  The reference's Model classes (Model.hpp:74,
// models/TinyYoloV2.hpp:93, DSCNNTiny.hpp, Resnet8Tiny.hpp, MobileNetTiny.hpp) run a network as a
// sequence of Layer::compute_output() calls, each of which ends in the layer functions of this
// platform; on a GPU every one of them is a kernel launch from the host.  capture() runs the
// callable once as it is (so that buffers are on the device and filters are re-laid where the
// tensor-core convolution wants them: nothing is left to allocate), then once more with this
// thread's layer calls recorded into a graph; launch() replays the recorded kernels on the same
// buffers with one call.  Whatever the callable returned in the recorded run (the model's output
// tensors) is where every replay leaves its results.  Combine with BatchScope for a batch.
//     small::b200::InferenceGraph g;
//     std::vector<small::Tensor<BufferT>*> out;
//     g.capture([&] { out = model.inference(&input); });
//     g.launch(); ... out[0]->buffer()[i]   // host access waits for the device
// The callable must only enqueue layer calls: host access to a buffer inside it throws.
class InferenceGraph
{
public:
    InferenceGraph() : m_stream(nullptr), m_exec(nullptr) { throw_on(small_b200_stream_create(&m_stream)); }
    InferenceGraph(InferenceGraph const &) = delete;
    InferenceGraph &operator=(InferenceGraph const &) = delete;
    ~InferenceGraph()
    {
        small_b200_device_sync();
        if (m_exec)
            small_b200_graph_destroy(m_exec);
        small_b200_stream_destroy(m_stream);
    }

    template <class Callable>
    void capture(Callable &&run)
    {
        if (m_exec)
        {
            throw_on(small_b200_device_sync());
            throw_on(small_b200_graph_destroy(m_exec));
            m_exec = nullptr;
        }
        run();
        flush_deferred();
        throw_on(small_b200_device_sync());
        pending() = false;
        StreamScope on(m_stream);
        throw_on(small_b200_graph_begin(m_stream));
        capturing() = true;
        try
        {
            run();
            flush_deferred();
        }
        catch (...)
        {
            deferred().valid = false;
            capturing() = false;
            void *dead = nullptr;
            small_b200_graph_end(m_stream, &dead); // ends the capture; its graph is discarded
            if (dead)
                small_b200_graph_destroy(dead);
            throw;
        }
        capturing() = false;
        throw_on(small_b200_graph_end(m_stream, &m_exec));
        pending() = false; // the recorded run launched nothing
    }

    bool captured() const { return m_exec != nullptr; }

    void launch()
    {
        if (!m_exec)
            throw std::logic_error("small::b200::InferenceGraph::launch before capture");
        flush_deferred();
        throw_on(small_b200_graph_launch(m_exec, m_stream));
        pending() = true;
    }

    void sync() { throw_on(small_b200_stream_sync(m_stream)); }

private:
    void *m_stream, *m_exec;
};
} // namespace b200

//****************************************************************************
class FloatBuffer : public b200::ManagedArray<float>
{
public:
    static uint32_t const W_ob{FLOAT_W_ob};
    static uint32_t const C_ob{FLOAT_C_ob};
    static uint32_t const SIMD{FLOAT_SIMD};
    static uint32_t const UNROLL{FLOAT_UNROLL};
    static uint32_t const C_ib{FLOAT_C_ib};
    static uint32_t const NUM_FMA{FLOAT_NUM_FMA};
    static uint32_t const NUM_MAX{FLOAT_NUM_MAX};
    static uint32_t const NUM_LOAD{FLOAT_NUM_LOAD};
    static uint32_t const NUM_STORE{FLOAT_NUM_STORE};

    typedef float value_type;
    typedef float accum_type;

    using b200::ManagedArray<float>::ManagedArray;
    FloatBuffer() = default;

    void swap(FloatBuffer &other) { b200::ManagedArray<float>::swap(other); }
    inline accum_type zero() const { return (accum_type)0; }
};

//****************************************************************************
class QUInt8Buffer : public b200::ManagedArray<uint8_t>
{
public:
    static uint32_t const W_ob{QUINT8_W_ob};
    static uint32_t const C_ob{QUINT8_C_ob};
    static uint32_t const SIMD{QUINT8_SIMD};
    static uint32_t const UNROLL{QUINT8_UNROLL};
    static uint32_t const C_ib{QUINT8_C_ib};
    static uint32_t const NUM_FMA{QUINT8_NUM_FMA};
    static uint32_t const NUM_MAX{QUINT8_NUM_MAX};
    static uint32_t const NUM_LOAD{QUINT8_NUM_LOAD};
    static uint32_t const NUM_STORE{QUINT8_NUM_STORE};

    typedef uint8_t value_type;
    typedef int32_t accum_type;

    QUInt8Buffer() : b200::ManagedArray<uint8_t>() { quantized_init(); }
    explicit QUInt8Buffer(size_t num_elts) : b200::ManagedArray<uint8_t>(num_elts) { quantized_init(); }
    QUInt8Buffer(QUInt8Buffer const &) = default;
    QUInt8Buffer &operator=(QUInt8Buffer const &) = default;

    QUInt8Buffer(QUInt8Buffer &&other) noexcept : b200::ManagedArray<uint8_t>()
    {
        quantized_init();
        swap(other);
    }
    QUInt8Buffer &operator=(QUInt8Buffer &&other) noexcept
    {
        if (this != &other)
        {
            QUInt8Buffer empty;
            swap(empty); // releases this buffer's storage when `empty` dies
            swap(other);
        }
        return *this;
    }

    void swap(QUInt8Buffer &other)
    {
        if (this == &other)
            return;
        b200::ManagedArray<uint8_t>::swap(other);
        std::swap(scale, other.scale);
        std::swap(offset, other.offset);
        std::swap(multiplier, other.multiplier);
        std::swap(lshift, other.lshift);
        std::swap(rshift, other.rshift);
        std::swap(m_zero, other.m_zero);
        std::swap(min_val, other.min_val);
        std::swap(max_val, other.max_val);
        std::swap(b, other.b);
    }

    inline accum_type zero() const { return m_zero; }

public:
    float scale;
    int32_t offset;
    int32_t multiplier;
    int lshift;
    int rshift;
    accum_type m_zero;
    int min_val;
    int max_val;
    uint8_t b;

private:
    // Parameters for the range [-1, 1] over 8 bits: the same fixed-point construction as
    // the reference's buffers (multiplier 1077952576, rshift 6, zero 128).
    void quantized_init()
    {
        b = 8;
        const double levels = 255.0;
        const double dscale = 2.0 / levels + 1e-17;
        int shift = 0;
        const double q = std::frexp(dscale, &shift);
        long long q_fixed = std::llround(q * (double)(1LL << 31));
        if (q_fixed == (1LL << 31))
        {
            q_fixed /= 2;
            ++shift;
        }
        if (shift < -31)
        {
            shift = 0;
            q_fixed = 0;
        }
        if (shift > 30)
        {
            shift = 30;
            q_fixed = (1LL << 31) - 1;
        }
        multiplier = (int32_t)q_fixed;
        m_zero = (accum_type)std::rint(levels / 2.0);
        scale = (float)dscale;
        lshift = shift > 0 ? shift : 0;
        rshift = shift > 0 ? 0 : -shift;
        min_val = 0;
        max_val = 255;
        offset = 0;
    }
};

//****************************************************************************
template <class BufferT>
inline BufferT *alloc_buffer(size_t num_elts)
{
    static_assert(std::is_same_v<BufferT, FloatBuffer> || std::is_same_v<BufferT, QUInt8Buffer>,
                  "small::alloc_buffer: unsupported buffer type");
    return new BufferT(num_elts);
}

template <class BufferT>
inline void free_buffer(BufferT *buffer)
{
    delete buffer;
}

} // namespace small
