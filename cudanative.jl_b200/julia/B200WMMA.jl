# B200WMMA.jl -- the Julia side of libb200wmma.so.
#
# Host code stays in Julia: this module keeps the names and argument order of CUDAnative.WMMA
# (src/device/cuda/wmma.jl of CUDAnative.jl) and of the CuHostArray convention (src/array.jl) and
# forwards every operation to the C ABI of include/b200wmma.h with `ccall`.  Device pointers are
# CUDAdrv `CuPtr`s, which `ccall` passes as plain addresses (src/array.jl:15 of the reference).
#
# Julia is not part of the build image of this repository, so this file is shipped unexecuted; it
# is kept to one `ccall` per entry point so that it can be checked against the header by eye.
module B200WMMA

using CUDAdrv: CuPtr, CuStream, CuDefaultStream

const lib = get(ENV, "B200WMMA_LIB", "libb200wmma")

# ---- status handling ---------------------------------------------------------------------------
struct B200Error <: Exception
    status::Cint
    msg::String
end
Base.showerror(io::IO, e::B200Error) = print(io, "B200Error(", e.status, "): ", e.msg)

last_error() = unsafe_string(ccall((:b200_last_error, lib), Cstring, ()))
@inline function check(status::Cint)
    status == 0 || throw(B200Error(status, last_error()))
    return nothing
end

# ---- layouts, uses, config: same names as CUDAnative.WMMA --------------------------------------
abstract type FragmentLayout end
struct RowMajor <: FragmentLayout end
struct ColMajor <: FragmentLayout end
struct Unspecified <: FragmentLayout end
abstract type FragmentUse end
struct MatrixA <: FragmentUse end
struct MatrixB <: FragmentUse end
struct Accumulator <: FragmentUse end
struct Config{M, N, K, d_type} end

layout_code(::Type{ColMajor}) = Cint(0)
layout_code(::Type{RowMajor}) = Cint(1)
layout_code(::Type{L}) where {L} = error("Invalid layout for WMMA: $L")
type_code(::Type{Float16}) = Cint(0)
type_code(::Type{Float32}) = Cint(1)
type_code(::Type{T}) where {T} = error("Invalid element type for WMMA: $T")
use_code(::Type{MatrixA}) = Cint(0)
use_code(::Type{MatrixB}) = Cint(1)
use_code(::Type{Accumulator}) = Cint(2)
check_shape(M, N, K) = (M, N, K) == (16, 16, 16) || error("Invalid shape for WMMA: (M, N, K) = ($M, $N, $K)")

# A fragment is the whole warp's register image in device memory: 32 lanes x FS elements.  It owns that
# memory (allocated by alloc_fragment) and gives it back when the garbage collector drops it, as the
# reference's CuHostArray does (src/array.jl:33-35).
mutable struct Fragment{M, N, K, FS, T, L <: FragmentLayout, U <: FragmentUse}
    x::CuPtr{T}
    function Fragment{M, N, K, FS, T, L, U}(x::CuPtr{T}) where {M, N, K, FS, T, L <: FragmentLayout, U <: FragmentUse}
        f = new{M, N, K, FS, T, L, U}(x)
        finalizer(free_fragment, f)
        return f
    end
end
free_fragment(f::Fragment) = ccall((:b200_free, lib), Cint, (CuPtr{Cvoid},), f.x)

num_elems(::Type{MatrixA}) = 16
num_elems(::Type{MatrixB}) = 16
num_elems(::Type{Accumulator}) = 8

function alloc_fragment(::Type{T}, fs) where {T}
    p = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:b200_malloc, lib), Cint, (Ptr{Ptr{Cvoid}}, Csize_t), p, 32 * fs * sizeof(T)))
    return reinterpret(CuPtr{T}, p[])
end

for (name, U) in ((:load_a, MatrixA), (:load_b, MatrixB), (:load_c, Accumulator))
    @eval function $name(addr::CuPtr{T}, stride::Number, ::Type{L}, ::Type{Config{M, N, K, D}};
                         stream::CuStream = CuDefaultStream()) where {T, L, M, N, K, D}
        check_shape(M, N, K)
        fs = num_elems($U)
        frag = alloc_fragment(T, fs)
        check(ccall((:b200_wmma_load, lib), Cint,
                    (Ptr{Cvoid}, Cint, Cint, Cint, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}),
                    stream.handle, use_code($U), layout_code(L), type_code(T), addr, stride, frag))
        Lret = $U === Accumulator ? Unspecified : L
        return Fragment{M, N, K, fs, T, Lret, $U}(frag)
    end
end

function fill_c(value::T, ::Type{Config{M, N, K, D}}; stream::CuStream = CuDefaultStream()) where {T, M, N, K, D}
    check_shape(M, N, K)
    frag = alloc_fragment(T, 8)
    check(ccall((:b200_wmma_fill_c, lib), Cint, (Ptr{Cvoid}, Cint, Cfloat, CuPtr{Cvoid}),
                stream.handle, type_code(T), Float32(value), frag))
    return Fragment{M, N, K, 8, T, Unspecified, Accumulator}(frag)
end

function mma(a::Fragment{M, N, K, 16, Float16, AL, MatrixA}, b::Fragment{M, N, K, 16, Float16, BL, MatrixB},
             c::Fragment{M, N, K, 8, CT, Unspecified, Accumulator}, ::Type{Config{M, N, K, DT}};
             stream::CuStream = CuDefaultStream()) where {M, N, K, AL, BL, CT, DT}
    check_shape(M, N, K)
    d = alloc_fragment(DT, 8)
    check(ccall((:b200_wmma_mma, lib), Cint,
                (Ptr{Cvoid}, Cint, Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}),
                stream.handle, type_code(CT), type_code(DT), a.x, b.x, c.x, d))
    return Fragment{M, N, K, 8, DT, Unspecified, Accumulator}(d)
end

function store_d(addr::CuPtr{T}, d::Fragment{M, N, K, 8, T, Unspecified, Accumulator}, stride::Number,
                 ::Type{L}, ::Type{Config{M, N, K, T}}; stream::CuStream = CuDefaultStream()) where {T, M, N, K, L}
    check(ccall((:b200_wmma_store_d, lib), Cint, (Ptr{Cvoid}, Cint, Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, Int64),
                stream.handle, layout_code(L), type_code(T), addr, d.x, stride))
    return nothing
end

# `alpha .* frag` and `alpha .+ frag` (wmma.jl:678-716): elementwise in the fragment's type
function bcast(op::Cint, s::Number, f::Fragment{M, N, K, FS, T, L, U}) where {M, N, K, FS, T, L, U}
    out = alloc_fragment(T, FS)
    check(ccall((:b200_wmma_bcast, lib), Cint, (Ptr{Cvoid}, Cint, Cint, Cint, Cfloat, CuPtr{Cvoid}, CuPtr{Cvoid}),
                C_NULL, op, type_code(T), FS, Float32(s), f.x, out))
    return Fragment{M, N, K, FS, T, L, U}(out)
end
Base.broadcasted(::typeof(*), s::Number, f::Fragment) = bcast(Cint(0), s, f)
Base.broadcasted(::typeof(+), s::Number, f::Fragment) = bcast(Cint(1), s, f)

# ---- the whole unit and the tiled GEMM ------------------------------------------------------------
"d = mma(alpha .* load_a(a), load_b(b), beta .* load_c(c)) in one launch (examples/wmma/high-level.jl:30-44)."
function wmma_16x16x16!(d::CuPtr{DT}, a::CuPtr{Float16}, b::CuPtr{Float16}, c::Union{CuPtr{CT}, Nothing};
                        a_layout = ColMajor, b_layout = ColMajor, c_layout = ColMajor, d_layout = ColMajor,
                        alpha = nothing, beta = nothing, lda = 16, ldb = 16, ldc = 16, ldd = 16, lowering = 0,
                        stream::CuStream = CuDefaultStream()) where {DT, CT}
    check(ccall((:b200_wmma_16x16x16, lib), Cint,
                (Ptr{Cvoid}, Cint, Cint, Cint, Cint, Cint, Cint, Cint, Cint, Cint, Cfloat, Cint, Cfloat,
                 CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64),
                stream.handle, lowering, layout_code(a_layout), layout_code(b_layout), layout_code(c_layout),
                layout_code(d_layout), c === nothing ? type_code(DT) : type_code(CT), type_code(DT),
                c === nothing ? 0 : 1, alpha === nothing ? 0 : 1, alpha === nothing ? 0f0 : Float32(alpha),
                beta === nothing ? 0 : 1, beta === nothing ? 0f0 : Float32(beta),
                a, lda, b, ldb, c === nothing ? CuPtr{Cvoid}(0) : c, ldc, d, ldd))
end

mutable struct Handle
    ptr::Ptr{Cvoid}
    function Handle(device::Integer = 0)
        p = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:b200_create, lib), Cint, (Ptr{Ptr{Cvoid}}, Cint), p, device))
        h = new(p[])
        finalizer(x -> ccall((:b200_destroy, lib), Cint, (Ptr{Cvoid},), x.ptr), h)
        return h
    end
end

"Set one of the B200_OPT_* options of include/b200wmma.h (kernel choice, tile width, split-K, wait budget ...)."
set_option!(h::Handle, option::Integer, value::Integer) =
    check(ccall((:b200_set_option, lib), Cint, (Ptr{Cvoid}, Cint, Int64), h.ptr, option, value))

"""
    device_status(h) -> (code, block, detail)

Reads (and clears) the device status word after a synchronisation: `code == 0` means no bounded wait inside a
kernel ran out -- the role of the reference's exception flag check (src/exceptions.jl:76-89).
"""
function device_status(h::Handle)
    code, block, detail = Ref{Cint}(0), Ref{Cint}(0), Ref{Cint}(0)
    check(ccall((:b200_device_status, lib), Cint, (Ptr{Cvoid}, Ptr{Cint}, Ptr{Cint}, Ptr{Cint}), h.ptr, code, block, detail))
    return (code[], block[], detail[])
end

"""
    gemm!(h, D, A, B, C; alpha = 1f0, beta = 0f0, transA = false, transB = false, stream)

`D = alpha * op(A) * op(B) + beta * C` on column-major device matrices given as (CuPtr, rows, cols, ld)
named tuples -- the multi-tile form of load_a / load_b / load_c -> mma -> store_d.
"""
function gemm!(h::Handle, D, A, B, C = nothing; alpha = 1f0, beta = 0f0, transA = false, transB = false,
               stream::CuStream = CuDefaultStream())
    M, K = transA ? (A.cols, A.rows) : (A.rows, A.cols)
    N = transB ? B.rows : B.cols
    check(ccall((:b200_gemm_f16f32, lib), Cint,
                (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Cfloat, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64,
                 Cfloat, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64),
                h.ptr, stream.handle, transA, transB, M, N, K, alpha, A.ptr, A.ld, B.ptr, B.ld, beta,
                C === nothing ? CuPtr{Cvoid}(0) : C.ptr, C === nothing ? M : C.ld, D.ptr, D.ld))
end

# element tags of include/b200wmma.h; bfloat16 data is passed as 16-bit words (e.g. CuPtr{UInt16})
const ELEM_F16, ELEM_F32, ELEM_BF16 = Cint(0), Cint(1), Cint(2)

"""
    gemm_strided_batched!(h, D, A, B, C; batch, ab_type, c_type, d_type, alpha, beta, transA, transB, stream)

`batch` products of one shape in one call (b200_gemm_strided_batched).  Operands are named tuples
(ptr, rows, cols, ld, stride): matrix i starts `stride * i` elements after `ptr`; a stride of 0 repeats
A, B or C.  `ab_type` is ELEM_F16 or ELEM_BF16, `c_type` / `d_type` any of the three tags.
`batch = 1` is b200_gemm_ex: one product with bfloat16 operands and / or 16-bit C and D.
"""
function gemm_strided_batched!(h::Handle, D, A, B, C = nothing; batch = 1, ab_type = ELEM_F16, c_type = ELEM_F32,
                               d_type = ELEM_F32, alpha = 1f0, beta = 0f0, transA = false, transB = false,
                               stream::CuStream = CuDefaultStream())
    M, K = transA ? (A.cols, A.rows) : (A.rows, A.cols)
    N = transB ? B.rows : B.cols
    check(ccall((:b200_gemm_strided_batched, lib), Cint,
                (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Cfloat, CuPtr{Cvoid}, Int64, Int64,
                 CuPtr{Cvoid}, Int64, Int64, Cint, Cfloat, CuPtr{Cvoid}, Int64, Int64, Cint, CuPtr{Cvoid}, Int64, Int64,
                 Cint, Int64),
                h.ptr, stream.handle, transA, transB, M, N, K, alpha, A.ptr, A.ld, A.stride, B.ptr, B.ld, B.stride,
                ab_type, beta, C === nothing ? CuPtr{Cvoid}(0) : C.ptr, C === nothing ? M : C.ld,
                C === nothing ? 0 : C.stride, c_type, D.ptr, D.ld, D.stride, d_type, batch))
end

"Host-buffer form: `Array`s in, `Array` out, copies inside (b200_gemm_f16f32_host)."
function gemm_host!(h::Handle, D::Matrix{Float32}, A::Matrix{Float16}, B::Matrix{Float16},
                    C::Union{Matrix{Float32}, Nothing} = nothing; alpha = 1f0, beta = 0f0, transA = false, transB = false)
    M, K = transA ? reverse(size(A)) : size(A)
    N = transB ? size(B, 1) : size(B, 2)
    check(ccall((:b200_gemm_f16f32_host, lib), Cint,
                (Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Cfloat, Ptr{Float16}, Int64, Ptr{Float16}, Int64, Cfloat,
                 Ptr{Float32}, Int64, Ptr{Float32}, Int64),
                h.ptr, transA, transB, M, N, K, alpha, A, stride(A, 2), B, stride(B, 2), beta,
                C === nothing ? C_NULL : C, C === nothing ? M : stride(C, 2), D, stride(D, 2)))
    return D
end

"""
    gemm_typed!(h, D, A, B, C; c_type, d_type, ...)

`gemm!` with Float16 or Float32 C and D chosen independently (b200_gemm_f16_typed): the four accumulator / result
type combinations of `Config{16, 16, 16, d_type}` and `load_c` (src/device/cuda/wmma.jl:23-30).
"""
function gemm_typed!(h::Handle, D, A, B, C = nothing; c_type = ELEM_F32, d_type = ELEM_F32, alpha = 1f0, beta = 0f0,
                     transA = false, transB = false, stream::CuStream = CuDefaultStream())
    M, K = transA ? (A.cols, A.rows) : (A.rows, A.cols)
    N = transB ? B.rows : B.cols
    check(ccall((:b200_gemm_f16_typed, lib), Cint,
                (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Cfloat, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64,
                 Cfloat, CuPtr{Cvoid}, Int64, Cint, CuPtr{Cvoid}, Int64, Cint),
                h.ptr, stream.handle, transA, transB, M, N, K, alpha, A.ptr, A.ld, B.ptr, B.ld, beta,
                C === nothing ? CuPtr{Cvoid}(0) : C.ptr, C === nothing ? M : C.ld, c_type, D.ptr, D.ld, d_type))
end

"""
    gemm_gated!(h, D, A, B, C, panel_flags, panel_k; ...)

`gemm!` whose main loop reads columns `[j*panel_k, (j+1)*panel_k)` of A only once the 32-bit device word
`panel_flags[j]` is non-zero (b200_gemm_f16f32_gated): one launch that overlaps the arrival of A.
"""
function gemm_gated!(h::Handle, D, A, B, C, panel_flags::CuPtr{UInt32}, panel_k::Integer; alpha = 1f0, beta = 0f0,
                     transA = false, transB = false, stream::CuStream = CuDefaultStream())
    M, K = transA ? (A.cols, A.rows) : (A.rows, A.cols)
    N = transB ? B.rows : B.cols
    check(ccall((:b200_gemm_f16f32_gated, lib), Cint,
                (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Cfloat, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64,
                 Cfloat, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64, CuPtr{UInt32}, Int64),
                h.ptr, stream.handle, transA, transB, M, N, K, alpha, A.ptr, A.ld, B.ptr, B.ld, beta,
                C === nothing ? CuPtr{Cvoid}(0) : C.ptr, C === nothing ? M : C.ld, D.ptr, D.ld, panel_flags, panel_k))
end

# ---- the allocation-free split-K product (no handle) -------------------------------------------------
"Once per device at start-up: address lookup and kernel loading for `gemm_splitk_static!` (b200_static_warmup)."
static_warmup() = check(ccall((:b200_static_warmup, lib), Cint, ()))

"`(code, block, detail)` of the static entry point's device status word; clears it (b200_static_status)."
function static_status()
    code, block, detail = Ref{Cint}(0), Ref{Cint}(0), Ref{Cint}(0)
    check(ccall((:b200_static_status, lib), Cint, (Ptr{Cint}, Ptr{Cint}, Ptr{Cint}), code, block, detail))
    return (code[], block[], detail[])
end

"""
    gemm_splitk_static!(D, A, B, C; split_k, sync = true, ...)

The product for callers that must not allocate device memory when they need it (b200_gemm_f16f32_splitk_static):
partial products live in a 16 MiB array inside the library image; calls on one device must not overlap.
"""
function gemm_splitk_static!(D, A, B, C = nothing; split_k = 2, sync = true, alpha = 1f0, beta = 0f0, transA = false,
                             transB = false, stream::CuStream = CuDefaultStream())
    M, K = transA ? (A.cols, A.rows) : (A.rows, A.cols)
    N = transB ? B.rows : B.cols
    check(ccall((:b200_gemm_f16f32_splitk_static, lib), Cint,
                (Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Cfloat, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64, Cfloat,
                 CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64, Cint, Cint),
                stream.handle, transA, transB, M, N, K, alpha, A.ptr, A.ld, B.ptr, B.ld, beta,
                C === nothing ? CuPtr{Cvoid}(0) : C.ptr, C === nothing ? M : C.ld, D.ptr, D.ld, split_k, sync ? 1 : 0))
end

# ---- N-sharded multi-GPU GEMM: one Julia process (or task) per device ------------------------------
const SHARDED_BLOB_BYTES = 128
const SHARDED_GATED, SHARDED_NO_TRANSFER = Cint(1), Cint(2)

"""
    Sharded(h, rank, world, M, N, K; panels = 16, exchange)

One rank of `D[:, slab_r] = alpha * A * B[:, slab_r] + beta * C[:, slab_r]` (b200_sharded_*).  `exchange` takes this
rank's 128-byte blob and returns the concatenation of every rank's blobs in rank order, e.g.
`blob -> MPI.Allgather(blob, comm)`.  `s.a` is this rank's A buffer (M x K Float16, valid on rank 0 before a product,
everywhere after it); `s.n0:s.n1-1` (0-based) are this rank's columns of B, C and D.
"""
mutable struct Sharded
    ptr::Ptr{Cvoid}
    a::CuPtr{Float16}
    n0::Int64
    n1::Int64
    function Sharded(h::Handle, rank::Integer, world::Integer, M::Integer, N::Integer, K::Integer; panels::Integer = 16,
                     exchange = nothing)
        p = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:b200_sharded_create, lib), Cint, (Ptr{Ptr{Cvoid}}, Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Cint),
                    p, h.ptr, rank, world, M, N, K, panels))
        n0, n1 = Ref{Int64}(0), Ref{Int64}(0)
        a, flags = Ref{Ptr{Cvoid}}(C_NULL), Ref{Ptr{Cvoid}}(C_NULL)
        np, ng = Ref{Cint}(0), Ref{Cint}(0)
        check(ccall((:b200_sharded_info, lib), Cint,
                    (Ptr{Cvoid}, Ptr{Int64}, Ptr{Int64}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Cint}, Ptr{Cint}),
                    p[], n0, n1, a, flags, np, ng))
        if world > 1
            blob = zeros(UInt8, SHARDED_BLOB_BYTES)
            check(ccall((:b200_sharded_ipc_blob, lib), Cint, (Ptr{Cvoid}, Ptr{UInt8}), p[], blob))
            blobs = exchange(blob)::Vector{UInt8}
            length(blobs) == world * SHARDED_BLOB_BYTES || error("exchange must return one 128-byte blob per rank")
            check(ccall((:b200_sharded_attach, lib), Cint, (Ptr{Cvoid}, Ptr{UInt8}), p[], blobs))
        end
        s = new(p[], reinterpret(CuPtr{Float16}, a[]), n0[], n1[])
        finalizer(x -> ccall((:b200_sharded_destroy, lib), Cint, (Ptr{Cvoid},), x.ptr), s)
        return s
    end
end

"Enqueue one product on `stream` (b200_sharded_run); every rank must make the call."
function run!(s::Sharded, D_slab, B_slab, C_slab = nothing; alpha = 1f0, beta = 0f0, flags = Cint(0),
              stream::CuStream = CuDefaultStream())
    check(ccall((:b200_sharded_run, lib), Cint,
                (Ptr{Cvoid}, Ptr{Cvoid}, Cfloat, CuPtr{Cvoid}, Int64, Cfloat, CuPtr{Cvoid}, Int64, CuPtr{Cvoid}, Int64, Cint),
                s.ptr, stream.handle, alpha, B_slab.ptr, B_slab.ld, beta,
                C_slab === nothing ? CuPtr{Cvoid}(0) : C_slab.ptr, C_slab === nothing ? D_slab.ld : C_slab.ld,
                D_slab.ptr, D_slab.ld, flags))
end

"Host-side wait with a deadline (b200_sharded_wait): throws B200Error(6, ...) when a peer never wrote its flags."
wait!(s::Sharded, timeout_ms::Integer = 60000) = check(ccall((:b200_sharded_wait, lib), Cint, (Ptr{Cvoid}, Int64), s.ptr, timeout_ms))

end # module
