export layer_norm!, layer_norm, ∇layer_norm!, ∇layer_norm

"`y = (x − μ) · rstd · w + b` per column of `X (M,N)` (biased variance); `W, B (M,)`."
function layer_norm!(Y, X, W, B; eps, TILE_M = 256, checkpoints = nothing)
    px, pw, pb, py = primal(X), primal(W), primal(B), primal(Y)
    M, N = size(px)
    @assert size(py) == (M, N)
    @assert size(pw) == (M,) && size(pb) == (M,)
    Mean = checkpoints === nothing ? nothing : get(checkpoints, :Mean, nothing)
    Rstd = checkpoints === nothing ? nothing : get(checkpoints, :Rstd, nothing)
    require_dense(px, pw, pb, py, Mean, Rstd)
    check(ccall((:tylo_b200_layer_norm_fwd, libtylo), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Float32, Int32, Ptr{Cvoid}),
                devptr(py), devptr(px), devptr(pw), devptr(pb), devptr(Mean), devptr(Rstd), M, N, Float32(eps),
                tylo_dtype(eltype(px)), current_stream()))
    return
end

allocate_checkpoints(::typeof(layer_norm!), X, W, B) =
    (; Mean = similar(W, Float32, size(X, 2)), Rstd = similar(W, Float32, size(X, 2)))

function layer_norm(X, W, B; eps, kwargs...)
    Y = similar(X)
    layer_norm!(Y, X, W, B; eps, kwargs...)
    return Y
end

"Backward of `layer_norm!`: overwrites `X.shadow`, `W.shadow`, `B.shadow`."
function ∇layer_norm!(Y::Duplicated, X::Duplicated, W::Duplicated, B::Duplicated; N_GROUPS = DEFAULT_N_GROUPS,
                      TILE_M = 256, TILE_F = 64, TILE_G = 64, checkpoints,
                      scratch = allocate_scratchspace(∇layer_norm!, primal(X), primal(W), primal(B); N_GROUPS))
    px, pw = primal(X), primal(W)
    M, N = size(px)
    PW, PB = scratch.W̄_partial, scratch.B̄_partial
    require_dense(px, pw, shadow(Y), shadow(X), shadow(W), shadow(B), PW, PB, checkpoints.Mean, checkpoints.Rstd)
    check(ccall((:tylo_b200_layer_norm_bwd, libtylo), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
                 Ptr{Cvoid}, Int32, Int64, Int64, Int32, Ptr{Cvoid}),
                devptr(shadow(X)), devptr(shadow(W)), devptr(shadow(B)), devptr(shadow(Y)), devptr(px), devptr(pw),
                devptr(checkpoints.Mean), devptr(checkpoints.Rstd), devptr(PW), devptr(PB), Int32(size(PW, 2)), M, N,
                tylo_dtype(eltype(px)), current_stream()))
    return
end

function allocate_scratchspace(::typeof(∇layer_norm!), X, W, B; N_GROUPS = DEFAULT_N_GROUPS)
    M, _ = size(X)
    return (; W̄_partial = similar(W, Float32, M, N_GROUPS), B̄_partial = similar(W, Float32, M, N_GROUPS),
              Locks = similar(X, Int, 0))
end

function ∇layer_norm(Ȳ::AbstractMatrix, X::AbstractMatrix, W::AbstractVector, B::AbstractVector; checkpoints,
                     N_GROUPS = DEFAULT_N_GROUPS, kwargs...)
    Xd, Wd, Bd = Duplicated(X), Duplicated(W), Duplicated(B)
    ∇layer_norm!(Duplicated(Ȳ, Ȳ), Xd, Wd, Bd; N_GROUPS, checkpoints)
    return shadow(Xd), shadow(Wd), shadow(Bd)
end
