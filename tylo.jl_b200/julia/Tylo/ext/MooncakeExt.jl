module MooncakeExt

# Mooncake reaches the kernels two ways.  The array-only entry points reuse the ChainRules rules
# (`@from_rrule`).  The all-positional flex core gets a rule of its own, because `@from_rrule` drops the
# tangent of struct arguments and a score mod with learnable parameters (ALiBi slopes, a bias table,
# a pair projection) is exactly such a struct.  Rules are registered over `AbstractFloat` element
# types, not `IEEEFloat`, so that BFloat16 arrays hit them too.

using Tylo
import Tylo: _flex_attention_core, grad_shadow, shadow, ScoreMod, MaskMod
using Mooncake
using Mooncake: DefaultCtx, @from_rrule, @is_primitive, CoDual, NoRData, NoFData, FData, primal, tangent, fdata,
    zero_tangent, lazy_zero_rdata, instantiate, increment!!
import Mooncake: rrule!!

const FloatArray{N} = AbstractArray{<:AbstractFloat,N}

@from_rrule DefaultCtx Tuple{typeof(rms_norm),FloatArray{2},FloatArray{1}} true
@from_rrule DefaultCtx Tuple{typeof(layer_norm),FloatArray{2},FloatArray{1},FloatArray{1}} true
@from_rrule DefaultCtx Tuple{typeof(softmax),FloatArray{2}} false
@from_rrule DefaultCtx Tuple{typeof(attention),FloatArray{4},FloatArray{4},FloatArray{4}} true
# keyword form of flex attention: gradients for Q, K, V only (the mods are fixed configuration there)
@from_rrule DefaultCtx Tuple{typeof(flex_attention),FloatArray{4},FloatArray{4},FloatArray{4}} true

# Adds a score mod's gradient shadow into the forward data Mooncake keeps for that mod: arrays are
# incremented in place, fields without a tangent are skipped, nested mods recurse field by field.
add_mod_grads!(acc::AbstractArray, g::AbstractArray) = (increment!!(acc, g); nothing)
add_mod_grads!(::NoFData, _) = nothing
function add_mod_grads!(acc::FData, g)
    for name in keys(acc.data)
        add_mod_grads!(getfield(acc.data, name), getfield(g, name))
    end
    return nothing
end

@is_primitive DefaultCtx Tuple{typeof(_flex_attention_core),FloatArray{4},FloatArray{4},FloatArray{4},ScoreMod,MaskMod,NamedTuple}

function rrule!!(::CoDual{typeof(_flex_attention_core)}, Q::CoDual, K::CoDual, V::CoDual, score::CoDual, mask::CoDual,
                 cfg::CoDual)
    q, k, v = primal(Q), primal(K), primal(V)
    score_mod, mask_mod, kw = primal(score), primal(mask), primal(cfg)
    cp = Tylo.allocate_checkpoints(flex_attention!, q, k, v)
    O = similar(q, size(v, 1), size(q, 2), size(q, 3), size(q, 4))
    flex_attention!(O, q, k, v; score_mod, mask_mod, checkpoints = cp, kw...)
    sc = Tylo.allocate_scratchspace(∇flex_attention!, q, k, v, O)
    Ō = fdata(zero_tangent(O))                  # whoever consumes O adds its cotangent here
    zeros_r = map(lazy_zero_rdata, (q, k, v, score_mod, mask_mod, kw))

    function flex_core_pullback(::NoRData)
        Qd, Kd, Vd = Duplicated(q), Duplicated(k), Duplicated(v)
        ∂mod = grad_shadow(score_mod)
        ∇flex_attention!(Duplicated(O, Ō), Qd, Kd, Vd; score_mod, mask_mod, ∂score_mod = ∂mod, checkpoints = cp,
                         scratch = sc, kw...)
        increment!!(tangent(Q), shadow(Qd))
        increment!!(tangent(K), shadow(Kd))
        increment!!(tangent(V), shadow(Vd))
        add_mod_grads!(tangent(score), ∂mod)
        return (NoRData(), map(instantiate, zeros_r)...)
    end
    return CoDual(O, Ō), flex_core_pullback
end

end
