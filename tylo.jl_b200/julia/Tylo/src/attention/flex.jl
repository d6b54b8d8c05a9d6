export flex_attention!, flex_attention, ∇flex_attention!, ∇flex_attention

"""
    flex_attention!(O, Q, K, V; score_mod = NoOpScore(), mask_mod = FullMask(), block_sparse = true,
                    input_pos = 0, qk_scale = nothing, checkpoints = nothing, kwargs...)

Attention with a score mod applied to the scaled scores and a mask mod (natural-base statistics;
a fully masked query gives `O = 0`, `M = -Inf`, `L = 0`).  Supported mods: `CausalMask`,
`SlidingWindowMask`, `DocumentMask`, `PrefixMask`, `prefix_lm` and their `&`; `SoftCapScore`,
`AliBiScore`, `BiasScore`, `PairFeatureScore` (evaluated into a bias table first) and their `∘`; anything
else throws `ArgumentError`.  With `block_mask`
(a `BlockMask` from `build_block_mask`) the forward walks the host-built block list instead of the
analytic block range; `TILE_M` / `TILE_N` are the edges the mask was built with (multiples of 32).
`tensorcore = TFloat32` on `Float32` arrays: TF32 operands on the tensor cores (head dims up to 64).
"""
function flex_attention!(O, Q, K, V; score_mod = NoOpScore(), mask_mod = FullMask(), block_mask = nothing,
                         block_sparse = true, input_pos = 0, qk_scale = nothing, tensorcore = nothing,
                         TILE_M = 64, TILE_N = 64, checkpoints = nothing)
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    Dk, Dv, Sq, Sk, H, Hkv, B = attn_dims(pQ, pK, pV)
    @assert size(pO) == (Dv, Sq, H, B)
    M = checkpoints === nothing ? nothing : get(checkpoints, :M, nothing)
    L = checkpoints === nothing ? nothing : get(checkpoints, :L, nothing)
    require_dense(pO, pQ, pK, pV, M, L)
    md, md_chain = describe_mask(mask_mod)
    score_mod = has_pairs(score_mod) ? lower_pairs(score_mod) : score_mod     # pair features run as bias tables
    sd = describe(score_mod)
    if block_mask isa BlockMask
        bm = block_mask
        @assert length(bm.count) == cld(Sq, TILE_M) && size(bm.idx) == size(bm.full) && size(bm.idx, 2) == length(bm.count)
        GC.@preserve score_mod mask_mod md_chain bm begin
            check(ccall((:tylo_b200_flex_attention_fwd_block_mask, libtylo), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ref{MaskDesc}, Ref{ScoreDesc},
                 Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Int32, Int32,
                 Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Float32, Int32, Ptr{Cvoid}),
                devptr(pO), devptr(pQ), devptr(pK), devptr(pV), devptr(M), devptr(L), md, sd,
                devptr(bm.count), devptr(bm.idx), devptr(bm.full), Int32(size(bm.idx, 1)), Int32(TILE_M), Int32(TILE_N),
                Dk, Dv, Sq, Sk, H, Hkv, B, Int32(input_pos), qk_scale === nothing ? 0.0f0 : Float32(qk_scale),
                fwd_dtype(eltype(pQ), tensorcore), current_stream()))
        end
        return
    end
    GC.@preserve score_mod mask_mod md_chain begin
        check(ccall((:tylo_b200_flex_attention_fwd, libtylo), Int32,
            (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ref{MaskDesc}, Ref{ScoreDesc},
             Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Float32, Int32, Int32, Ptr{Cvoid}),
            devptr(pO), devptr(pQ), devptr(pK), devptr(pV), devptr(M), devptr(L), md, sd,
            Dk, Dv, Sq, Sk, H, Hkv, B, Int32(input_pos), qk_scale === nothing ? 0.0f0 : Float32(qk_scale),
            Int32(block_sparse), fwd_dtype(eltype(pQ), tensorcore), current_stream()))
    end
    return
end

allocate_checkpoints(::typeof(flex_attention!), Q, K, V) = allocate_checkpoints(attention!, Q, K, V)

# The AD rules differentiate these two: `_flex_attention` exposes the score mod as a positional
# argument (its parameters can receive gradients), `_flex_attention_core` takes everything positionally.
function _flex_attention_core(Q, K, V, score_mod, mask_mod, cfg::NamedTuple)
    O = similar(Q, size(V, 1), size(Q, 2), size(Q, 3), size(Q, 4))
    flex_attention!(O, Q, K, V; score_mod, mask_mod, cfg...)
    return O
end
_flex_attention(Q, K, V, score_mod; mask_mod = FullMask(), kwargs...) =
    _flex_attention_core(Q, K, V, score_mod, mask_mod, NamedTuple(kwargs))
"Allocating forward; the autodiff entry point."
flex_attention(Q, K, V; score_mod = NoOpScore(), kwargs...) = _flex_attention(Q, K, V, score_mod; kwargs...)

"""
    ∇flex_attention!(O, Q, K, V::Duplicated…; score_mod, mask_mod, ∂score_mod = nothing, checkpoints, scratch = …)

Backward of `flex_attention!` (overwrites the input shadows).  `∂score_mod = grad_shadow(score_mod)`
accumulates score-mod parameter gradients (ALiBi slopes).
"""
function ∇flex_attention!(O::Duplicated, Q::Duplicated, K::Duplicated, V::Duplicated; score_mod = NoOpScore(),
                          mask_mod = FullMask(), ∂score_mod = nothing, block_mask = nothing, block_sparse = true,
                          input_pos = 0, qk_scale = nothing, tensorcore = nothing, TILE_M = 64, TILE_N = 64, checkpoints,
                          scratch = allocate_scratchspace(∇flex_attention!, primal(Q), primal(K), primal(V), primal(O)))
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    Dk, Dv, Sq, Sk, H, Hkv, B = attn_dims(pQ, pK, pV)
    @assert size(pO, 1) == Dv
    (; M, L) = checkpoints
    Δ = scratch.Δ
    ws = get(scratch, :workspace, nothing)
    ws === nothing && (ws = bwd_workspace(pQ, pK, pV))
    require_dense(pO, pQ, pK, pV, shadow(O), shadow(Q), shadow(K), shadow(V), M, L, Δ, ws)
    md, md_chain = describe_mask(mask_mod)
    pair_mod, ∂pair_mod = score_mod, ∂score_mod
    if has_pairs(score_mod)               # pair features run as bias tables; their gradients are folded back below
        score_mod = lower_pairs(pair_mod)
        ∂score_mod = lower_pair_shadows(score_mod, ∂pair_mod)
    end
    sd = describe(score_mod, ∂score_mod)
    if block_mask isa BlockMask          # gradients of the block-list forward (an extension: upstream has none)
        bm = block_mask
        GC.@preserve score_mod mask_mod md_chain ∂score_mod bm begin
            check(ccall((:tylo_b200_flex_attention_bwd_block_mask, libtylo), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
                 Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Ref{MaskDesc}, Ref{ScoreDesc},
                 Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Int32, Int32,
                 Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Float32, Int32, Ptr{Cvoid}),
                devptr(shadow(Q)), devptr(shadow(K)), devptr(shadow(V)), devptr(pQ), devptr(pK), devptr(pV), devptr(pO),
                devptr(shadow(O)), devptr(M), devptr(L), devptr(Δ), devptr(ws), Int64(length(ws)), md, sd,
                devptr(bm.count), devptr(bm.idx), devptr(bm.full), Int32(size(bm.idx, 1)), Int32(TILE_M), Int32(TILE_N),
                Dk, Dv, Sq, Sk, H, Hkv, B, Int32(input_pos), qk_scale === nothing ? 0.0f0 : Float32(qk_scale),
                tylo_dtype(eltype(pQ)), current_stream()))
        end
        ∂pair_mod === nothing || raise_pair_grads!(∂pair_mod, pair_mod, ∂score_mod)
        return
    end
    GC.@preserve score_mod mask_mod md_chain ∂score_mod begin
        check(ccall((:tylo_b200_flex_attention_bwd, libtylo), Int32,
            (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
             Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Ref{MaskDesc}, Ref{ScoreDesc},
             Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Float32, Int32, Int32, Ptr{Cvoid}),
            devptr(shadow(Q)), devptr(shadow(K)), devptr(shadow(V)), devptr(pQ), devptr(pK), devptr(pV), devptr(pO),
            devptr(shadow(O)), devptr(M), devptr(L), devptr(get(scratch, :Ō′, nothing)), devptr(Δ), devptr(ws),
            Int64(length(ws)), md, sd, Dk, Dv, Sq, Sk, H, Hkv, B, Int32(input_pos),
            qk_scale === nothing ? 0.0f0 : Float32(qk_scale), Int32(block_sparse), tylo_dtype(eltype(pQ)),
            current_stream()))
    end
    ∂pair_mod === nothing || raise_pair_grads!(∂pair_mod, pair_mod, ∂score_mod)
    return
end

allocate_scratchspace(::typeof(∇flex_attention!), Q, K, V, O; kwargs...) =
    allocate_scratchspace(∇attention!, Q, K, V, O; kwargs...)

"Allocating backward: `(Q̄, K̄, V̄)`."
function ∇flex_attention(Ō, Q, K, V, O; checkpoints, kwargs...)
    Qd, Kd, Vd = Duplicated(Q), Duplicated(K), Duplicated(V)
    ∇flex_attention!(Duplicated(O, Ō), Qd, Kd, Vd; checkpoints, kwargs...)
    return shadow(Qd), shadow(Kd), shadow(Vd)
end
