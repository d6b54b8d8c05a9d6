export softmax!, softmax, ∇softmax!, ∇softmax

"Numerically stable softmax over each column (dim 1) of `X`, written to `Y`.  Returns `nothing`."
function softmax!(Y, X)
    px, py = primal(X), primal(Y)
    M, N = size(px)
    @assert size(py) == (M, N)
    require_dense(px, py)
    check(ccall((:tylo_b200_softmax_fwd, libtylo), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int32, Ptr{Cvoid}),
                devptr(py), devptr(px), M, N, tylo_dtype(eltype(px)), current_stream()))
    return
end

function softmax(X)
    Y = similar(X)
    softmax!(Y, X)
    return Y
end

"Backward from the forward output: `X.shadow = y ∘ (ȳ − Σ y∘ȳ)` (overwrite).  Returns `nothing`."
function ∇softmax!(Y::Duplicated, X::Duplicated)
    py = primal(Y)
    M, N = size(py)
    require_dense(py, shadow(Y), shadow(X))
    check(ccall((:tylo_b200_softmax_bwd, libtylo), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int32, Ptr{Cvoid}),
                devptr(shadow(X)), devptr(shadow(Y)), devptr(py), M, N, tylo_dtype(eltype(py)), current_stream()))
    return
end

function ∇softmax(Ȳ, Y)
    Xd = Duplicated(Y, similar(Y))      # only the shadow is written
    ∇softmax!(Duplicated(Y, Ȳ), Xd)
    return shadow(Xd)
end
