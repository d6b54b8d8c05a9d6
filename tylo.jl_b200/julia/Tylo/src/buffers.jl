export Duplicated, allocate_checkpoints, allocate_scratchspace
public primal, shadow

"""
    Duplicated(primal, shadow)
    Duplicated(x)

An array together with the buffer that receives its gradient.  The backward entry points
(`∇f!`) read primals and the output's shadow and OVERWRITE the input shadows.  Forward entry
points accept either a bare array or a `Duplicated` (only the primal is read).
`Duplicated(x)` allocates an uninitialised shadow like `x`.
"""
struct Duplicated{P,S}
    primal::P
    shadow::S
end
Duplicated(x) = Duplicated(x, similar(x))

"`x` itself, or the primal of a `Duplicated`."
@inline primal(x) = x
@inline primal(d::Duplicated) = d.primal

"The gradient buffer of a `Duplicated`."
@inline shadow(d::Duplicated) = d.shadow

"""
    allocate_checkpoints(f!, args...) -> NamedTuple

Saved activations that bridge `f!` and `∇f!` (`(; M, L)` for attention, `(; Rstd)` for RMSNorm,
`(; Mean, Rstd)` for LayerNorm); always `Float32`.  Pass as the `checkpoints` keyword.
"""
function allocate_checkpoints end

"""
    allocate_scratchspace(f!, args...; kw...) -> NamedTuple

Transient workspace of one pass.  Pass as the `scratch` keyword; reusing one allocation across
calls keeps the library allocation-free (it never allocates device memory itself).
"""
function allocate_scratchspace end
