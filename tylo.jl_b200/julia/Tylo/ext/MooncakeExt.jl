module MooncakeExt

# Mooncake reaches the kernels through the ChainRules rules.  The rules are registered over
# AbstractFloat element types (not IEEEFloat) so that BFloat16 arrays hit them too.

using Tylo
import Tylo: _flex_attention, _flex_attention_core, grad_shadow, ScoreMod, MaskMod
using Mooncake, ChainRulesCore
import Mooncake: @from_rrule, DefaultCtx

const FloatArray{N} = AbstractArray{<:AbstractFloat,N}

@from_rrule DefaultCtx Tuple{typeof(rms_norm),FloatArray{2},FloatArray{1}} true
@from_rrule DefaultCtx Tuple{typeof(layer_norm),FloatArray{2},FloatArray{1},FloatArray{1}} true
@from_rrule DefaultCtx Tuple{typeof(softmax),FloatArray{2}} false
@from_rrule DefaultCtx Tuple{typeof(attention),FloatArray{4},FloatArray{4},FloatArray{4}} true
@from_rrule DefaultCtx Tuple{typeof(flex_attention),FloatArray{4},FloatArray{4},FloatArray{4}} true

# `_flex_attention_core(Q, K, V, score_mod, mask_mod, cfg)` is the all-positional form Mooncake
# differentiates when score-mod parameters (ALiBi slopes) need gradients; it forwards to the
# ChainRules rule of `_flex_attention`.
function ChainRulesCore.rrule(::typeof(_flex_attention_core), Q, K, V, score_mod::ScoreMod, mask_mod::MaskMod, cfg::NamedTuple)
    O, back = ChainRulesCore.rrule(_flex_attention, Q, K, V, score_mod; mask_mod, cfg...)
    pullback(Ō) = (back(Ō)..., ChainRulesCore.NoTangent(), ChainRulesCore.NoTangent())
    return O, pullback
end
@from_rrule DefaultCtx Tuple{typeof(_flex_attention_core),FloatArray{4},FloatArray{4},FloatArray{4},ScoreMod,MaskMod,NamedTuple} false

end
