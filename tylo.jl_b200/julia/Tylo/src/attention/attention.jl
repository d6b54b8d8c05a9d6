export attention!, attention, ∇attention!, ∇attention

function attn_dims(pQ, pK, pV)
    Dq, Sq, H, B = size(pQ)
    Dk, Sk, Hkv, Bk = size(pK)
    Dv, Sv, Hv, Bv = size(pV)
    @assert Dq == Dk
    @assert Sk == Sv
    @assert Hkv == Hv
    @assert B == Bk == Bv
    @assert iszero(H % Hkv)
    eltype(pQ) === eltype(pK) === eltype(pV) || throw(ArgumentError("Q, K, V must share one element type"))
    return Int32.((Dk, Dv, Sq, Sk, H, Hkv, B))
end

"""
    attention!(O, Q, K, V; causal = false, input_pos = 0, k_lengths = nothing, q_lengths = nothing,
               checkpoints = nothing, kwargs...)

Fused multi-head attention with GQA.  `Q (Dk,Sq,H,B)`, `K (Dk,Sk,Hkv,B)`, `V (Dv,Sk,Hkv,B)`,
`O (Dv,Sq,H,B)`; scale `1/√Dk`.  `checkpoints = allocate_checkpoints(attention!, Q, K, V)` saves the
softmax statistics for `∇attention!`.  `TILE_M`, `TILE_N` are accepted for source compatibility and ignored
(tile shapes are fixed per kernel).  `Float32` arrays are computed in true fp32 unless `tensorcore = TFloat32`
asks for TF32 operands on the tensor cores (head dims up to 64).
Returns `nothing`.
"""
function attention!(O, Q, K, V; causal = false, input_pos = 0, k_lengths = nothing, q_lengths = nothing,
                    tensorcore = nothing, TILE_M = 64, TILE_N = 64, checkpoints = nothing)
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    Dk, Dv, Sq, Sk, H, Hkv, B = attn_dims(pQ, pK, pV)
    @assert size(pO) == (Dv, Sq, H, B)
    M = checkpoints === nothing ? nothing : get(checkpoints, :M, nothing)
    L = checkpoints === nothing ? nothing : get(checkpoints, :L, nothing)
    require_dense(pO, pQ, pK, pV, M, L, k_lengths, q_lengths)
    check(ccall((:tylo_b200_attention_fwd, libtylo), Int32,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Ptr{Cvoid}),
        devptr(pO), devptr(pQ), devptr(pK), devptr(pV), devptr(M), devptr(L), devptr(k_lengths), devptr(q_lengths),
        Dk, Dv, Sq, Sk, H, Hkv, B, Int32(input_pos), Int32(causal), fwd_dtype(eltype(pQ), tensorcore), current_stream()))
    return
end

"`(; M, L)`: per-query row max (log2 units) and row sum, `(Sq, H, B)` `Float32`."
allocate_checkpoints(::typeof(attention!), Q, K, V) =
    (; M = similar(Q, Float32, (size(Q, 2), size(Q, 3), size(Q, 4))),
       L = similar(Q, Float32, (size(Q, 2), size(Q, 3), size(Q, 4))))

"Allocating forward; the autodiff entry point."
function attention(Q, K, V; kwargs...)
    O = similar(Q, size(V, 1), size(Q, 2), size(Q, 3), size(Q, 4))
    attention!(O, Q, K, V; kwargs...)
    return O
end

function bwd_workspace(Q, K, V)
    Dk, Dv, Sq, Sk, H, Hkv, B = attn_dims(Q, K, V)
    n = ccall((:tylo_b200_attention_bwd_workspace_bytes, libtylo), Int64,
              (Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32), Dk, Dv, Sq, Sk, H, Hkv, B, tylo_dtype(eltype(Q)))
    return similar(Q, UInt8, max(n, 16))
end

"""
    ∇attention!(O::Duplicated, Q::Duplicated, K::Duplicated, V::Duplicated; causal, checkpoints, scratch = …)

Backward of `attention!`: reads `O.shadow` and the primals, overwrites `Q.shadow`, `K.shadow`,
`V.shadow`.  `causal` / `input_pos` must match the forward.  Returns `nothing`.
"""
function ∇attention!(O::Duplicated, Q::Duplicated, K::Duplicated, V::Duplicated; causal, input_pos = 0,
                     k_lengths = nothing, q_lengths = nothing, tensorcore = nothing, TILE_M = 64, TILE_N = 64,
                     checkpoints,
                     scratch = allocate_scratchspace(∇attention!, primal(Q), primal(K), primal(V), primal(O)))
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    Dk, Dv, Sq, Sk, H, Hkv, B = attn_dims(pQ, pK, pV)
    @assert size(pO, 1) == Dv
    @assert size(shadow(O), 1) == Dv
    (; M, L) = checkpoints
    Δ = scratch.Δ
    ws = get(scratch, :workspace, nothing)
    ws === nothing && (ws = bwd_workspace(pQ, pK, pV))
    require_dense(pO, pQ, pK, pV, shadow(O), shadow(Q), shadow(K), shadow(V), M, L, Δ, ws)
    check(ccall((:tylo_b200_attention_bwd, libtylo), Int32,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Ptr{Cvoid}, Ptr{Cvoid},
         Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Ptr{Cvoid}),
        devptr(shadow(Q)), devptr(shadow(K)), devptr(shadow(V)), devptr(pQ), devptr(pK), devptr(pV), devptr(pO),
        devptr(shadow(O)), devptr(M), devptr(L), devptr(get(scratch, :Ō′, nothing)), devptr(Δ), devptr(ws),
        Int64(length(ws)), devptr(k_lengths), devptr(q_lengths),
        Dk, Dv, Sq, Sk, H, Hkv, B, Int32(input_pos), Int32(causal), tylo_dtype(eltype(pQ)), current_stream()))
    return
end

"`(; Ō′, Δ, workspace)`: `Ō′` is kept for source compatibility (unused), `Δ` is `(Sq,H,B)` `Float32`."
function allocate_scratchspace(::typeof(∇attention!), Q, K, V, O; kwargs...)
    return (; Ō′ = similar(O, 0), Δ = similar(O, Float32, (size(O, 2), size(O, 3), size(O, 4))),
              workspace = bwd_workspace(Q, K, V))
end

"Allocating backward: `(Q̄, K̄, V̄)`."
function ∇attention(Ō, Q, K, V, O; checkpoints, causal, kwargs...)
    Qd, Kd, Vd = Duplicated(Q), Duplicated(K), Duplicated(V)
    ∇attention!(Duplicated(O, Ō), Qd, Kd, Vd; checkpoints, causal, kwargs...)
    return shadow(Qd), shadow(Kd), shadow(Vd)
end
