module ChainRulesCoreExt

# Reverse rules for the allocating entry points.  Each rule runs the in-place forward with freshly
# allocated checkpoints, allocates the backward scratch once, and returns a pullback that calls the
# in-place backward — so a captured graph of forward + pullback reuses all memory.

using Tylo
import Tylo: shadow, _flex_attention, grad_shadow, ScoreMod
using ChainRulesCore
import ChainRulesCore: rrule, unthunk, NoTangent, Tangent

function rrule(::typeof(rms_norm), X, W; eps, offset = 0.0f0)
    cp = allocate_checkpoints(rms_norm!, X, W)
    Y = similar(X)
    rms_norm!(Y, X, W; eps, offset, checkpoints = cp)
    sc = allocate_scratchspace(∇rms_norm!, X, W)
    function pullback(Ȳ)
        Xd, Wd = Duplicated(X), Duplicated(W)
        ∇rms_norm!(Duplicated(Y, unthunk(Ȳ)), Xd, Wd; offset, checkpoints = cp, scratch = sc)
        return NoTangent(), shadow(Xd), shadow(Wd)
    end
    return Y, pullback
end

function rrule(::typeof(layer_norm), X, W, B; eps)
    cp = allocate_checkpoints(layer_norm!, X, W, B)
    Y = similar(X)
    layer_norm!(Y, X, W, B; eps, checkpoints = cp)
    sc = allocate_scratchspace(∇layer_norm!, X, W, B)
    function pullback(Ȳ)
        Xd, Wd, Bd = Duplicated(X), Duplicated(W), Duplicated(B)
        ∇layer_norm!(Duplicated(Y, unthunk(Ȳ)), Xd, Wd, Bd; checkpoints = cp, scratch = sc)
        return NoTangent(), shadow(Xd), shadow(Wd), shadow(Bd)
    end
    return Y, pullback
end

function rrule(::typeof(softmax), X)
    Y = softmax(X)
    function pullback(Ȳ)
        Xd = Duplicated(X)
        ∇softmax!(Duplicated(Y, unthunk(Ȳ)), Xd)
        return NoTangent(), shadow(Xd)
    end
    return Y, pullback
end

function rrule(::typeof(attention), Q, K, V; causal = false, kwargs...)
    cp = allocate_checkpoints(attention!, Q, K, V)
    O = similar(Q, size(V, 1), size(Q, 2), size(Q, 3), size(Q, 4))
    attention!(O, Q, K, V; causal, checkpoints = cp, kwargs...)
    sc = allocate_scratchspace(∇attention!, Q, K, V, O)
    function pullback(Ō)
        Qd, Kd, Vd = Duplicated(Q), Duplicated(K), Duplicated(V)
        ∇attention!(Duplicated(O, unthunk(Ō)), Qd, Kd, Vd; causal, checkpoints = cp, scratch = sc, kwargs...)
        return NoTangent(), shadow(Qd), shadow(Kd), shadow(Vd)
    end
    return O, pullback
end

# gradients with respect to Q, K, V only
function rrule(::typeof(flex_attention), Q, K, V; kwargs...)
    cp = allocate_checkpoints(flex_attention!, Q, K, V)
    O = similar(Q, size(V, 1), size(Q, 2), size(Q, 3), size(Q, 4))
    flex_attention!(O, Q, K, V; checkpoints = cp, kwargs...)
    sc = allocate_scratchspace(∇flex_attention!, Q, K, V, O)
    function pullback(Ō)
        Qd, Kd, Vd = Duplicated(Q), Duplicated(K), Duplicated(V)
        ∇flex_attention!(Duplicated(O, unthunk(Ō)), Qd, Kd, Vd; checkpoints = cp, scratch = sc, kwargs...)
        return NoTangent(), shadow(Qd), shadow(Kd), shadow(Vd)
    end
    return O, pullback
end

# A gradient shadow (the mod's own struct type, arrays holding gradients, everything else carried along
# unchanged) as a ChainRules tangent: arrays are their own tangent, nested mods become a `Tangent` over
# their field names, plain fields (head counts, caps, ops) have none.  Works for every score mod, so a
# `BiasScore` table or the projection of a `PairFeatureScore` receives its gradient like ALiBi slopes do.
score_tangent(x::AbstractArray) = x
score_tangent(m::ScoreMod) = Tangent{typeof(m)}(; (f => score_tangent(getfield(m, f)) for f in fieldnames(typeof(m)))...)
score_tangent(::Any) = NoTangent()

# gradients with respect to Q, K, V and the score mod's parameters
function rrule(::typeof(_flex_attention), Q, K, V, score_mod::ScoreMod; mask_mod = Tylo.FullMask(), kwargs...)
    cp = allocate_checkpoints(flex_attention!, Q, K, V)
    O = similar(Q, size(V, 1), size(Q, 2), size(Q, 3), size(Q, 4))
    flex_attention!(O, Q, K, V; score_mod, mask_mod, checkpoints = cp, kwargs...)
    sc = allocate_scratchspace(∇flex_attention!, Q, K, V, O)
    function pullback(Ō)
        Qd, Kd, Vd = Duplicated(Q), Duplicated(K), Duplicated(V)
        ∂mod = grad_shadow(score_mod)
        ∇flex_attention!(Duplicated(O, unthunk(Ō)), Qd, Kd, Vd; score_mod, mask_mod, ∂score_mod = ∂mod,
                         checkpoints = cp, scratch = sc, kwargs...)
        return NoTangent(), shadow(Qd), shadow(Kd), shadow(Vd), score_tangent(∂mod)
    end
    return O, pullback
end

end
