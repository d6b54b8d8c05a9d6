export decode_attention!

"A split count that fills the GPU for this cache (the reference's fixed 8 gives 8·Hkv·B blocks)."
suggest_splits(Sk, Hkv, B) =
    Int(ccall((:tylo_b200_decode_suggest_splits, libtylo), Int32, (Int32, Int32, Int32), Sk, Hkv, B))

"""
    decode_attention!(O, Q, K, V; lengths, n_splits = nothing, scratch = …) -> O

Split-KV attention for one query token per sequence.  `Q (Dk,H,B)`, `K (Dk,Sk,Hkv,B)`,
`V (Dv,Sk,Hkv,B)`, `O (Dv,H,B)`, `lengths` a device `Int32` vector of valid cache lengths.
`n_splits = nothing` lets the library choose; an explicit count (the reference's default is 8) is
honoured.  `TILE_N`, `tensorcore` are accepted and ignored.
"""
function decode_attention!(O, Q, K, V; lengths, tensorcore = nothing, TILE_N = 64, n_splits = nothing,
                           scratch = nothing)
    Dq, H, B = size(Q)
    Dk, Sk, Hkv, Bk = size(K)
    Dv, Sv, Hv, Bv = size(V)
    @assert Dq == Dk
    @assert Sk == Sv
    @assert Hkv == Hv
    @assert B == Bk == Bv
    @assert size(O) == (Dv, H, B)
    @assert iszero(H % Hkv)
    if scratch === nothing
        n_splits === nothing && (n_splits = suggest_splits(Sk, Hkv, B))
        scratch = allocate_scratchspace(decode_attention!, O, Q; n_splits)
    end
    (; O_partial, M_partial, L_partial) = scratch
    ns = size(O_partial, 4)
    eltype(lengths) === Int32 || throw(ArgumentError("lengths must be Int32"))
    require_dense(O, Q, K, V, lengths, O_partial, M_partial, L_partial)
    check(ccall((:tylo_b200_decode_attention, libtylo), Int32,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Ptr{Cvoid}),
        devptr(O), devptr(Q), devptr(K), devptr(V), devptr(lengths), devptr(O_partial), devptr(M_partial),
        devptr(L_partial), Int32(ns), Int32(Dk), Int32(Dv), Int32(Sk), Int32(H), Int32(Hkv), Int32(B),
        tylo_dtype(eltype(Q)), current_stream()))
    return O
end

"`(; O_partial (Dv,H,B,n_splits), M_partial, L_partial (H,B,n_splits))`, all `Float32`."
function allocate_scratchspace(::typeof(decode_attention!), O, Q; n_splits = 8)
    Dv, H, B = size(O)
    return (; O_partial = similar(O, Float32, (Dv, H, B, n_splits)),
              M_partial = similar(O, Float32, (H, B, n_splits)),
              L_partial = similar(O, Float32, (H, B, n_splits)))
end
