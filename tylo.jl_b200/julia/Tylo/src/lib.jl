# ccall plumbing shared by every wrapper.

const libtylo = get(ENV, "TYLO_B200_LIB", "libtylo_b200")

const BFloat16 = CUDACore.BFloat16

tylo_dtype(::Type{Float32}) = Int32(0)
tylo_dtype(::Type{BFloat16}) = Int32(1)
tylo_dtype(::Type{Float16}) = Int32(2)
tylo_dtype(T::Type) = throw(ArgumentError("libtylo_b200 has no kernels for element type $T"))

"""
    TFloat32

Value of the `tensorcore` keyword of `attention!` / `flex_attention!` that asks for both matrix products on the
tensor cores with TF32 operands for `Float32` arrays (the reference's default for `Float32`, utils.jl:43-44).
The default here, `tensorcore = nothing`, computes `Float32` in true fp32.  Forward only, head dims up to 64.
"""
struct TFloat32 end
export TFloat32

"Element-type code of a forward attention call: `Float32` arrays with `tensorcore = TFloat32` run as TF32."
fwd_dtype(T::Type, tensorcore) = (T === Float32 && is_tf32(tensorcore)) ? Int32(3) : tylo_dtype(T)
is_tf32(x::Type) = nameof(x) === :TFloat32        # this package's marker or another package's type of that name
is_tf32(x::Symbol) = x === :TFloat32 || x === :tf32
is_tf32(x) = false

# ---- the three version-dependent spellings -------------------------------------------------
"""
    devptr(a)

Raw device address of a dense device array (`C_NULL` for `nothing`).  Only arrays whose `pointer`
is a device pointer (`CuPtr`) are accepted: a host `Array` here would hand the kernel an address
the GPU cannot read, so it is refused with an `ArgumentError` before anything is launched.
"""
devptr(::Nothing) = Ptr{Cvoid}(C_NULL)
devptr(a::AbstractArray) = devptr(a, pointer(a))
devptr(a, p::CUDACore.CuPtr) = reinterpret(Ptr{Cvoid}, UInt(p))
devptr(a, p) = throw(ArgumentError(
    "libtylo_b200 reads device memory only: got a $(typeof(a)) whose pointer is a $(typeof(p)); move it to the GPU first (e.g. `CuArray(x)`)"))
devptr(a) = throw(ArgumentError("libtylo_b200 takes device arrays, got a $(typeof(a))"))
"Handle of the CUDA stream of the current task."
current_stream() = reinterpret(Ptr{Cvoid}, CUDACore.stream().handle)
"Whether `a` is a dense column-major array (views with gaps are not accepted)."
is_dense(a) = stride(a, 1) == 1 && all(stride(a, i + 1) == stride(a, i) * size(a, i) for i in 1:ndims(a)-1)
# ---------------------------------------------------------------------------------------------

function require_dense(arrays...)
    for a in arrays
        a === nothing && continue
        is_dense(a) || throw(ArgumentError("libtylo_b200 takes dense column-major arrays"))
    end
end

"Turn a library status into the exception the reference wrapper would have thrown."
function check(status::Int32)
    status == 0 && return nothing
    msg = unsafe_string(ccall((:tylo_b200_last_error, libtylo), Cstring, ()))
    status == 1 && throw(AssertionError(msg))        # the wrappers' @assert
    status == 2 && throw(ArgumentError(msg))         # unsupported by libtylo_b200 (no fallback)
    error("libtylo_b200 status $status: $msg")
end

"Synchronise and report whether a bounded device-side wait gave up (0 = healthy)."
function device_status()
    code = Ref{Int32}(0)
    check(ccall((:tylo_b200_device_status, libtylo), Int32, (Ref{Int32},), code))
    return code[]
end
