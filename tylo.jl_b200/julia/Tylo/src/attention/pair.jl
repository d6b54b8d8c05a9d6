export PairFeatureScore, pair_feature, ∇pair_feature

# Pair-feature bias: `s[kv, q] += Σ_p pair_proj[h, p] * φ_p`, with `φ = pair_feature(op, qvals, kvals)`
# computed from per-position feature vectors `qvals = q_features[:, q, b]`, `kvals = k_features[:, kv, b]`.
#
# `pair_feature` is user code.  libtylo_b200 cannot compile Julia into its kernels, so the bias is not
# fused: the wrappers evaluate the user's broadcast definition on whole feature rows with array
# broadcasts on the GPU, which yields the `(Sk, Sq, heads, batch)` table of a `BiasScore`, and the
# kernels run that.  Same results and same gradients as a fused evaluation, at the price of the table
# (`4·Sk·Sq·H·B` bytes) — for long sequences chunk the queries (`input_pos` does not shift features).

"""
    pair_feature(op, qvals::NTuple{F}, kvals::NTuple{F}) -> NTuple{PD}

The `PD` pair features of one (query, key) pair from its `F` feature values each.  Write the method
for your `op` type with dot broadcasts over the tuple entries: the entries are scalars when a mod is
evaluated on the host (`hscore`) and `(1, Sq)` / `(Sk, 1)` device arrays when the bias table is built,
and broadcasting lifts one definition to both.  There is no fallback method on purpose: a missing
implementation is a `MethodError`.
"""
function pair_feature end

"""
    ∇pair_feature(op, qvals, kvals, dphi::NTuple{PD}) -> (dq::NTuple{F}, dk::NTuple{F})

Vector-Jacobian product of [`pair_feature`](@ref), in the same broadcast style; every returned entry
must be a broadcast over the inputs (`0f0 .* qvals[f]` for a zero, not a bare scalar).  Needed only for
feature gradients (`grad_shadow(mod; feature_grads = true)`).
"""
function ∇pair_feature end

"""
    PairFeatureScore(op, q_features, k_features, pair_proj)

Adds `Σ_p pair_proj[h, p] * pair_feature(op, …)[p]` to the scores.  `q_features` is `(F, Sq, batch)`,
`k_features` `(F, Sk, batch)`, `pair_proj` `(heads, PD)`; features are indexed by local position.
"""
struct PairFeatureScore{F,PD,Op,AQ,AK,P} <: ScoreMod
    nfeat::Val{F}
    npair::Val{PD}
    op::Op
    q_features::AQ
    k_features::AK
    pair_proj::P
end

function PairFeatureScore(op, q_features::AbstractArray, k_features::AbstractArray, pair_proj::AbstractMatrix)
    F = Int(size(q_features, 1))
    size(k_features, 1) == F ||
        throw(DimensionMismatch("q_features has $F feature rows, k_features has $(size(k_features, 1))"))
    return PairFeatureScore(Val(F), Val(Int(size(pair_proj, 2))), op, q_features, k_features, pair_proj)
end

# host evaluation on scalars (0-based positions); use `adapt(Array, mod)` for device-resident features
function (m::PairFeatureScore{F,PD})(s, b, h, q::Integer, kv::Integer) where {F,PD}
    qvals = ntuple(f -> m.q_features[f, q+1, b], Val(F))
    kvals = ntuple(f -> m.k_features[f, kv+1, b], Val(F))
    phi = pair_feature(m.op, qvals, kvals)
    return s + sum(ntuple(p -> m.pair_proj[h, p] * phi[p], Val(PD)))
end

grad_shadow(m::PairFeatureScore; feature_grads::Bool = false) = PairFeatureScore(m.nfeat, m.npair, m.op,
    feature_grads ? fill!(similar(m.q_features), 0) : nothing,
    feature_grads ? fill!(similar(m.k_features), 0) : nothing,
    fill!(similar(m.pair_proj), 0))

# feature rows of batch entry `b` shaped for an outer-product broadcast: queries along dim 2, keys along dim 1
feature_rows(m::PairFeatureScore{F}, b) where {F} = (
    ntuple(f -> reshape(view(m.q_features, f, :, b), 1, :), Val(F)),
    ntuple(f -> reshape(view(m.k_features, f, :, b), :, 1), Val(F)))

"""
    pair_bias(m::PairFeatureScore) -> Array{Float32,4}  # (Sk, Sq, heads, batch), where the features live

The bias table the mod stands for, by array broadcasts of the user's `pair_feature`.
"""
function pair_bias(m::PairFeatureScore{F,PD}) where {F,PD}
    Sq, Sk, B = size(m.q_features, 2), size(m.k_features, 2), size(m.q_features, 3)
    proj = Array(m.pair_proj)                       # small; scalar reads happen on the host copy
    H = size(proj, 1)
    bias = similar(m.q_features, Float32, Sk, Sq, H, B)
    for b in 1:B
        qvals, kvals = feature_rows(m, b)
        phi = pair_feature(m.op, qvals, kvals)
        for h in 1:H
            dst = view(bias, :, :, h, b)
            dst .= Float32(proj[h, 1]) .* phi[1]
            for p in 2:PD
                dst .+= Float32(proj[h, p]) .* phi[p]
            end
        end
    end
    return bias
end

"""
    pair_grads!(∂m, m, d_bias)

Folds the bias-table gradient `d_bias` `(Sk, Sq, heads, batch)` the backward kernel produced into the
shadow `∂m`: `∂proj[h, p] += Σ d_bias[:, :, h, b] ∘ φ_p`, and, when `∂m` carries feature buffers,
the feature gradients through `∇pair_feature` (summed over keys for queries, over queries for keys).
"""
function pair_grads!(∂m::PairFeatureScore, m::PairFeatureScore{F,PD}, d_bias) where {F,PD}
    proj = Array(m.pair_proj)
    H, B = size(proj, 1), size(m.q_features, 3)
    dproj = zeros(Float32, H, PD)
    for b in 1:B
        qvals, kvals = feature_rows(m, b)
        phi = pair_feature(m.op, qvals, kvals)
        for h in 1:H
            s̄ = view(d_bias, :, :, h, b)
            for p in 1:PD
                dproj[h, p] += Float32(sum(s̄ .* phi[p]))
            end
            if ∂m.q_features !== nothing
                dphi = ntuple(p -> Float32(proj[h, p]) .* s̄, Val(PD))
                dq, dk = ∇pair_feature(m.op, qvals, kvals, dphi)
                for f in 1:F
                    view(∂m.q_features, f, :, b) .+= vec(sum(dq[f]; dims = 1))
                    view(∂m.k_features, f, :, b) .+= vec(sum(dk[f]; dims = 2))
                end
            end
        end
    end
    ∂m.pair_proj .+= typeof(∂m.pair_proj)(dproj)
    return ∂m
end

# ---- lowering of a score chain that contains pair-feature mods to the library's bias tables -----------
# `lower_pairs(mod)` returns the chain with every `PairFeatureScore` replaced by its `BiasScore`;
# `lower_pair_shadows` does the same for a gradient shadow (zeroed tables of the same size), and
# `raise_pair_grads!` folds those tables back after the backward call.
lower_pairs(m::ScoreMod) = m
lower_pairs(m::PairFeatureScore) = BiasScore(pair_bias(m))
lower_pairs(m::ComposeScore) = ComposeScore(lower_pairs(m.a), lower_pairs(m.b))

lower_pair_shadows(low, ∂m) = ∂m
lower_pair_shadows(low::BiasScore, ∂m::PairFeatureScore) = BiasScore(fill!(similar(low.bias), 0), low.nheads, low.nbatch)
lower_pair_shadows(low::ComposeScore, ∂m::ComposeScore) = ComposeScore(lower_pair_shadows(low.a, ∂m.a), lower_pair_shadows(low.b, ∂m.b))
lower_pair_shadows(low, ::Nothing) = nothing

raise_pair_grads!(∂m, m, ∂low) = nothing
raise_pair_grads!(∂m::PairFeatureScore, m::PairFeatureScore, ∂low::BiasScore) = pair_grads!(∂m, m, ∂low.bias)
function raise_pair_grads!(∂m::ComposeScore, m::ComposeScore, ∂low::ComposeScore)
    raise_pair_grads!(∂m.a, m.a, ∂low.a)
    raise_pair_grads!(∂m.b, m.b, ∂low.b)
    return nothing
end

has_pairs(::ScoreMod) = false
has_pairs(::PairFeatureScore) = true
has_pairs(m::ComposeScore) = has_pairs(m.a) || has_pairs(m.b)
