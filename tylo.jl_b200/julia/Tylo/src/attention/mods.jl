export FullMask, CausalMask, SlidingWindowMask, PrefixMask, DocumentMask
export AndMask, OrMask, prefix_lm
export NoOpScore, SoftCapScore, AliBiScore, BiasScore, ComposeScore
export hmask, hscore
export grad_shadow
export BlockMask, build_block_mask

# Score / mask mods.  The types, constructors and operators are the API; the device side is a set of
# compiled variants inside libtylo_b200 selected through two plain descriptors.  Calling a mod with
# scalars evaluates it on the host (the CPU reference for the exact mod the kernel runs).
# Positions are 0-based and absolute (queries are shifted by `input_pos`); `b`, `h` are 1-based.

abstract type MaskMod end
abstract type ScoreMod end

# `adapt(Array, mod)` gives a host-indexable copy of any mod (and `adapt(CuArray, mod)` the way back):
# the struct is rebuilt from its adapted fields, field-less mods come back as themselves.  This is how a
# mod that holds device arrays is evaluated with `hmask` / `hscore` without scalar-indexing the GPU.
function Adapt.adapt_structure(to, m::Union{MaskMod,ScoreMod})
    T = typeof(m)
    n = fieldcount(T)
    n == 0 && return m
    return T.name.wrapper((adapt(to, getfield(m, i)) for i in 1:n)...)
end

"Evaluate a mask mod on the host at scalar positions; for a mod that holds device arrays pass `adapt(Array, mod)`."
hmask(m::MaskMod, q, kv; b = 1, h = 1) = m(Int32(b), Int32(h), q, kv)
"Evaluate a score mod on the host for scalar score `s`; for a mod that holds device arrays pass `adapt(Array, mod)`."
hscore(m::ScoreMod, s, q, kv; b = 1, h = 1) = m(s, Int32(b), Int32(h), q, kv)

"No masking."
struct FullMask <: MaskMod end
(::FullMask)(b, h, q, kv) = true

"`q ≥ kv`."
struct CausalMask <: MaskMod end
(::CausalMask)(b, h, q, kv) = q >= kv

"Causal attention within a window: `q - w ≤ kv ≤ q`."
struct SlidingWindowMask <: MaskMod
    w::Int32
end
(m::SlidingWindowMask)(b, h, q, kv) = (q >= kv) & (q <= kv + m.w)

"Keys at `kv < len` are visible."
struct PrefixMask <: MaskMod
    len::Int32
end
(m::PrefixMask)(b, h, q, kv) = kv < m.len

"""
    DocumentMask(doc)            # one Int32 id per absolute position, shared by every batch entry
    DocumentMask(doc_q, doc_kv)

A pair attends iff its document ids match.  Extension over the reference: an `(S, B)` matrix
gives every batch entry its own id table.
"""
struct DocumentMask{A,B} <: MaskMod
    doc_q::A
    doc_kv::B
end
DocumentMask(doc::AbstractVecOrMat) = DocumentMask(doc, doc)
(m::DocumentMask)(b, h, q, kv) = ndims(m.doc_q) == 2 ? m.doc_q[q+1, b] == m.doc_kv[kv+1, b] : m.doc_q[q+1] == m.doc_kv[kv+1]

struct AndMask{A<:MaskMod,B<:MaskMod} <: MaskMod
    a::A
    b::B
end
(m::AndMask)(b, h, q, kv) = m.a(b, h, q, kv) & m.b(b, h, q, kv)

struct OrMask{A<:MaskMod,B<:MaskMod} <: MaskMod
    a::A
    b::B
end
(m::OrMask)(b, h, q, kv) = m.a(b, h, q, kv) | m.b(b, h, q, kv)

Base.:&(a::MaskMod, b::MaskMod) = AndMask(a, b)
Base.:|(a::MaskMod, b::MaskMod) = OrMask(a, b)

"Bidirectional over the first `len` positions, causal after."
prefix_lm(len) = CausalMask() | PrefixMask(Int32(len))

"""
    BlockMask(count, idx, full)

Host-built coarse block sparsity for `flex_attention!(…; block_mask)`: per query block the 0-based key
blocks that hold any unmasked pair (`idx[1:count[i], i]`) and whether each is fully unmasked
(`full`).  Device `Int32` arrays; forward only.
"""
struct BlockMask{C,I}
    count :: C    # [n_qb]
    idx   :: I    # [n_kb, n_qb]
    full  :: I    # [n_kb, n_qb]
end

"""
    build_block_mask(keep, n_q, n_kv; TILE_M = 64, TILE_N = 64, input_pos = 0, to_device = CuArray)

Evaluates `keep(q, kv)::Bool` (0-based absolute positions) once per pair on the host and lists, per
block of `TILE_M` queries, the blocks of `TILE_N` keys with any pair kept; a listed block is marked full
when every pair is kept and it does not touch the end of Q or K.  The three `Int32` arrays are moved to
the GPU with `to_device` (`CuArray` unless told otherwise), so the result can go straight into
`flex_attention!(…; block_mask)`; pass `to_device = identity` to keep host arrays for inspection.
"""
function build_block_mask(keep, n_q, n_kv; TILE_M::Int = 64, TILE_N::Int = 64, input_pos::Int = 0, to_device = CuArray)
    nqb, nkb = cld(n_q, TILE_M), cld(n_kv, TILE_N)
    idx, full, cnt = zeros(Int32, nkb, nqb), zeros(Int32, nkb, nqb), zeros(Int32, nqb)
    for i in 1:nqb
        qs = (i - 1) * TILE_M : min(i * TILE_M, n_q) - 1
        slot = 0
        for j in 1:nkb
            ks = (j - 1) * TILE_N : min(j * TILE_N, n_kv) - 1
            kept = count(keep(q + input_pos, kv)::Bool for q in qs, kv in ks)
            kept == 0 && continue
            slot += 1
            idx[slot, i] = j - 1
            full[slot, i] = (kept == length(qs) * length(ks) && i * TILE_M <= n_q && j * TILE_N <= n_kv) ? 1 : 0
        end
        cnt[i] = slot
    end
    BlockMask(to_device(cnt), to_device(idx), to_device(full))
end

struct NoOpScore <: ScoreMod end
(::NoOpScore)(s, b, h, q, kv) = s

"`s -> cap * tanh(s / cap)`."
struct SoftCapScore <: ScoreMod
    cap::Float32
end
(m::SoftCapScore)(s, b, h, q, kv) = m.cap * tanh(s / m.cap)

"`s + slopes[h] * (q - kv)`, one slope per query head."
struct AliBiScore{A} <: ScoreMod
    slopes::A
end
(m::AliBiScore)(s, b, h, q, kv) = s + m.slopes[h] * Float32(q - kv)

"Additive bias `(N_kv, M_q, heads, batch)`, `Float32`, indexed by local rows (not shifted by `input_pos`); heads and batch broadcast by `mod1`.  Runs on the library's fp32-arithmetic kernels."
struct BiasScore{A} <: ScoreMod
    bias::A
    nheads::Int32
    nbatch::Int32
end
BiasScore(bias::AbstractArray{<:Any,4}) = BiasScore(bias, Int32(size(bias, 3)), Int32(size(bias, 4)))
(m::BiasScore)(s, b, h, q, kv) = s + m.bias[kv+1, q+1, mod1(h, m.nheads), mod1(b, m.nbatch)]

"Apply `a`, then `b`; written `b ∘ a`."
struct ComposeScore{A<:ScoreMod,B<:ScoreMod} <: ScoreMod
    a::A
    b::B
end
(m::ComposeScore)(s, b, h, q, kv) = m.b(m.a(s, b, h, q, kv), b, h, q, kv)
Base.:∘(b::ScoreMod, a::ScoreMod) = ComposeScore(a, b)

"""
    grad_shadow(x)

Zeroed gradient accumulator: a zeroed copy of an array, or a score mod rebuilt with zeroed array
fields.  Pass a score-mod shadow as `∂score_mod` to `∇flex_attention!`; valid for one backward call.
"""
grad_shadow(x::AbstractArray) = fill!(similar(x), 0)
grad_shadow(m::AliBiScore) = AliBiScore(grad_shadow(m.slopes))
grad_shadow(m::BiasScore) = BiasScore(grad_shadow(m.bias), m.nheads, m.nbatch)
grad_shadow(m::ComposeScore) = ComposeScore(grad_shadow(m.a), grad_shadow(m.b))
grad_shadow(x) = x

# ---- descriptors handed to the library (layout of tylo_mask_desc / tylo_score_desc) -----------------
const MASK_CAUSAL = UInt32(1); const MASK_SLIDING = UInt32(2); const MASK_DOCUMENT = UInt32(4)
const MASK_PREFIX = UInt32(8); const MASK_PREFIX_LM = UInt32(16)
const SCORE_ALIBI = UInt32(1); const SCORE_SOFTCAP = UInt32(2); const SCORE_SOFTCAP_FIRST = UInt32(4)
const SCORE_BIAS = UInt32(8)

mutable struct MaskDesc
    flags::UInt32
    window::Int32
    prefix_len::Int32
    reserved::Int32
    doc_q::Ptr{Cvoid}
    doc_kv::Ptr{Cvoid}
    doc_batch_stride::Int64
    doc_q_len::Int64
    doc_kv_len::Int64
    or_next::Ptr{Cvoid}      # next conjunction of the disjunctive normal form, or C_NULL
end
MaskDesc() = MaskDesc(0, 0, 0, 0, C_NULL, C_NULL, 0, 0, 0, C_NULL)

mutable struct ScoreDesc
    flags::UInt32
    cap::Float32
    slopes::Ptr{Cvoid}
    d_slopes::Ptr{Cvoid}
    bias::Ptr{Cvoid}
    d_bias::Ptr{Cvoid}
    bias_heads::Int32
    bias_batch::Int32
end
ScoreDesc() = ScoreDesc(0, 1.0f0, C_NULL, C_NULL, C_NULL, C_NULL, 1, 1)

unsupported(what) = throw(ArgumentError("$what is unsupported by libtylo_b200 (there is no fallback)"))

describe!(d::MaskDesc, ::FullMask) = d
describe!(d::MaskDesc, ::CausalMask) = (d.flags |= MASK_CAUSAL; d)
function describe!(d::MaskDesc, m::SlidingWindowMask)
    d.window = (d.flags & MASK_SLIDING) != 0 ? min(d.window, m.w) : m.w
    d.flags |= MASK_SLIDING
    d
end
function describe!(d::MaskDesc, m::PrefixMask)
    (d.flags & MASK_PREFIX_LM) != 0 && unsupported("PrefixMask combined with prefix_lm")
    d.prefix_len = (d.flags & MASK_PREFIX) != 0 ? min(d.prefix_len, m.len) : m.len
    d.flags |= MASK_PREFIX
    d
end
function describe!(d::MaskDesc, m::DocumentMask)
    (d.flags & MASK_DOCUMENT) != 0 && unsupported("more than one DocumentMask")
    eltype(m.doc_q) === Int32 && eltype(m.doc_kv) === Int32 || throw(ArgumentError("DocumentMask ids must be Int32"))
    require_dense(m.doc_q, m.doc_kv)
    ndims(m.doc_q) == ndims(m.doc_kv) || throw(ArgumentError("doc_q and doc_kv must both be vectors or both matrices"))
    d.flags |= MASK_DOCUMENT
    d.doc_q = devptr(m.doc_q); d.doc_kv = devptr(m.doc_kv)
    d.doc_q_len = size(m.doc_q, 1); d.doc_kv_len = size(m.doc_kv, 1)
    if ndims(m.doc_q) == 2
        size(m.doc_q) == size(m.doc_kv) || throw(ArgumentError("per-batch id tables must share one size"))
        d.doc_batch_stride = size(m.doc_q, 1)
    end
    d
end
# prefix_lm(len) = CausalMask() | PrefixMask(len) stays ONE term of a conjunction (its own flag)
struct PrefixLMTerm <: MaskMod
    len::Int32
end
function describe!(d::MaskDesc, m::PrefixLMTerm)
    (d.flags & (MASK_PREFIX | MASK_PREFIX_LM)) != 0 && unsupported("prefix_lm combined with another prefix term")
    d.flags |= MASK_PREFIX_LM; d.prefix_len = m.len
    d
end
describe!(::MaskDesc, m::MaskMod) = unsupported("mask mod $(typeof(m))")

# Disjunctive normal form of a mask tree: a vector of conjunctions, each a vector of atomic masks.
clauses(::FullMask) = [MaskMod[]]
clauses(m::MaskMod) = [MaskMod[m]]
clauses(m::AndMask) = [vcat(a, b) for a in clauses(m.a) for b in clauses(m.b)]
function clauses(m::OrMask)
    a, b = m.a, m.b
    a isa PrefixMask && b isa CausalMask && return [MaskMod[PrefixLMTerm(a.len)]]
    b isa PrefixMask && a isa CausalMask && return [MaskMod[PrefixLMTerm(b.len)]]
    vcat(clauses(a), clauses(b))
end

const MAX_MASK_CLAUSES = 4

"""
    describe_mask(mask_mod) -> (first::MaskDesc, chain::Vector{MaskDesc})

The descriptors of the mask's conjunctions, linked through `or_next`.  `chain` must stay alive
(`GC.@preserve`) for the duration of the call that receives `first`.
"""
function describe_mask(mask_mod::MaskMod)
    cs = clauses(mask_mod)
    length(cs) <= MAX_MASK_CLAUSES || unsupported("a mask with $(length(cs)) OR-ed conjunctions")
    chain = [foldl(describe!, c; init = MaskDesc()) for c in cs]
    for i in 1:length(chain)-1
        chain[i].or_next = pointer_from_objref(chain[i+1])
    end
    return chain[1], chain
end

flatten(m::ComposeScore, ∂m) = vcat(flatten(m.a, ∂m === nothing ? nothing : ∂m.a), flatten(m.b, ∂m === nothing ? nothing : ∂m.b))
flatten(::NoOpScore, ∂m) = Tuple{ScoreMod,Any}[]
flatten(m::ScoreMod, ∂m) = Tuple{ScoreMod,Any}[(m, ∂m)]

function describe(score_mod::ScoreMod, ∂score_mod = nothing)
    d = ScoreDesc()
    chain = flatten(score_mod, ∂score_mod)
    # the additive mods (ALiBi, bias) share one place in the chain: all before or all after the soft cap
    caps = findall(x -> x[1] isa SoftCapScore, chain)
    adds = findall(x -> x[1] isa AliBiScore || x[1] isa BiasScore, chain)
    if !isempty(caps) && !isempty(adds) && !(maximum(adds) < caps[1] || minimum(adds) > caps[1])
        unsupported("additive score mods on both sides of a SoftCapScore")
    end
    for (i, (m, ∂m)) in enumerate(chain)
        if m isa SoftCapScore
            (d.flags & SCORE_SOFTCAP) != 0 && unsupported("more than one SoftCapScore")
            d.flags |= SCORE_SOFTCAP; d.cap = m.cap
            !isempty(adds) && minimum(adds) > i && (d.flags |= SCORE_SOFTCAP_FIRST)
        elseif m isa AliBiScore
            (d.flags & SCORE_ALIBI) != 0 && unsupported("more than one AliBiScore")
            eltype(m.slopes) === Float32 || throw(ArgumentError("AliBiScore slopes must be Float32"))
            d.flags |= SCORE_ALIBI; d.slopes = devptr(m.slopes)
            ∂m === nothing || (d.d_slopes = devptr(∂m.slopes))
        elseif m isa BiasScore
            (d.flags & SCORE_BIAS) != 0 && unsupported("more than one BiasScore")
            eltype(m.bias) === Float32 || throw(ArgumentError("BiasScore bias must be Float32"))
            d.flags |= SCORE_BIAS; d.bias = devptr(m.bias); d.bias_heads = m.nheads; d.bias_batch = m.nbatch
            ∂m === nothing || (d.d_bias = devptr(∂m.bias))
        else
            unsupported("score mod $(typeof(m))")
        end
    end
    d
end
