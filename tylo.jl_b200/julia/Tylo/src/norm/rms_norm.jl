export rms_norm!, rms_norm, ∇rms_norm!, ∇rms_norm

const DEFAULT_N_GROUPS = 296   # two CTAs per SM on a 148-SM part

"`y = x · rstd · (w + offset)`, `rstd = 1/√(mean(x²) + eps)` per column of `X (M,N)`; `W (M,)`."
function rms_norm!(Y, X, W; eps, offset = 0.0f0, TILE_M = 256, checkpoints = nothing)
    px, pw, py = primal(X), primal(W), primal(Y)
    M, N = size(px)
    @assert size(py) == (M, N)
    @assert size(pw) == (M,)
    Rstd = checkpoints === nothing ? nothing : get(checkpoints, :Rstd, nothing)
    require_dense(px, pw, py, Rstd)
    check(ccall((:tylo_b200_rms_norm_fwd, libtylo), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Float32, Float32, Int32, Ptr{Cvoid}),
                devptr(py), devptr(px), devptr(pw), devptr(Rstd), M, N, Float32(eps), Float32(offset),
                tylo_dtype(eltype(px)), current_stream()))
    return
end

allocate_checkpoints(::typeof(rms_norm!), X, W) = (; Rstd = similar(W, Float32, size(X, 2)))

function rms_norm(X, W; eps, offset = 0.0f0, kwargs...)
    Y = similar(X)
    rms_norm!(Y, X, W; eps, offset, kwargs...)
    return Y
end

"Backward of `rms_norm!`: overwrites `X.shadow`, `W.shadow`.  No locks are used; `scratch.Locks` is ignored."
function ∇rms_norm!(Y::Duplicated, X::Duplicated, W::Duplicated; offset = 0.0f0, N_GROUPS = DEFAULT_N_GROUPS,
                    TILE_M = 256, TILE_F = 64, TILE_G = 64, checkpoints,
                    scratch = allocate_scratchspace(∇rms_norm!, primal(X), primal(W); N_GROUPS))
    px, pw = primal(X), primal(W)
    M, N = size(px)
    P = scratch.W̄_partial
    require_dense(px, pw, shadow(Y), shadow(X), shadow(W), P, checkpoints.Rstd)
    check(ccall((:tylo_b200_rms_norm_bwd, libtylo), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Int64, Int64,
                 Float32, Int32, Ptr{Cvoid}),
                devptr(shadow(X)), devptr(shadow(W)), devptr(shadow(Y)), devptr(px), devptr(pw), devptr(checkpoints.Rstd),
                devptr(P), Int32(size(P, 2)), M, N, Float32(offset), tylo_dtype(eltype(px)), current_stream()))
    return
end

function allocate_scratchspace(::typeof(∇rms_norm!), X, W; N_GROUPS = DEFAULT_N_GROUPS)
    M, _ = size(X)
    return (; W̄_partial = similar(W, Float32, M, N_GROUPS), Locks = similar(X, Int, 0))
end

function ∇rms_norm(Ȳ::AbstractMatrix, X::AbstractMatrix, W::AbstractVector; checkpoints, offset = 0.0f0,
                   N_GROUPS = DEFAULT_N_GROUPS, kwargs...)
    Xd, Wd = Duplicated(X), Duplicated(W)
    ∇rms_norm!(Duplicated(Ȳ, Ȳ), Xd, Wd; offset, N_GROUPS, checkpoints)
    return shadow(Xd), shadow(Wd)
end
