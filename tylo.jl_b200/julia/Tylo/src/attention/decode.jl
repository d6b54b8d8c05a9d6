export decode_attention!, paged_decode_attention!, sharded_decode_attention!, DecodeExchange, exchange_status

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
    tickets = get(scratch, :tickets, nothing)      # scratch from older code has none: two launches then
    ns = size(O_partial, 4)
    eltype(lengths) === Int32 || throw(ArgumentError("lengths must be Int32"))
    require_dense(O, Q, K, V, lengths, O_partial, M_partial, L_partial, tickets)
    # one launch: the split kernel's last block per (kv head, batch) merges the partials itself
    check(ccall((:tylo_b200_decode_attention_fused, libtylo), Int32,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Ptr{Cvoid}),
        devptr(O), devptr(Q), devptr(K), devptr(V), devptr(lengths), devptr(O_partial), devptr(M_partial),
        devptr(L_partial), devptr(tickets), Int32(ns), Int32(Dk), Int32(Dv), Int32(Sk), Int32(H), Int32(Hkv), Int32(B),
        tylo_dtype(eltype(Q)), current_stream()))
    return O
end

"""
`(; O_partial (Dv,H,B,n_splits), M_partial, L_partial (H,B,n_splits))`, all `Float32`, as in the reference,
plus `tickets`: zeroed `Int32` counters of the one-launch form (the kernels leave them zero; one scratch must
not serve two calls that overlap on the GPU).
"""
function allocate_scratchspace(::typeof(decode_attention!), O, Q; n_splits = 8)
    Dv, H, B = size(O)
    nt = ccall((:tylo_b200_decode_ticket_count, libtylo), Int64, (Int32, Int32, Int32), n_splits, H, B)
    return (; O_partial = similar(O, Float32, (Dv, H, B, n_splits)),
              M_partial = similar(O, Float32, (H, B, n_splits)),
              L_partial = similar(O, Float32, (H, B, n_splits)),
              tickets = fill!(similar(O, Int32, (max(nt, 1),)), 0))
end

"""
    paged_decode_attention!(O, Q, K_pages, V_pages; block_table, lengths, n_splits = nothing, scratch = …) -> O

`decode_attention!` over a paged KV cache (no counterpart in the reference): `K_pages (Dk, page_size, Hkv, n_pages)`
and `V_pages (Dv, page_size, Hkv, n_pages)` are pools of pages, `block_table` a device `Int32` `(max_pages, B)`
matrix of 0-based page ids (keys `[i*page_size, (i+1)*page_size)` of sequence `b` live in page
`block_table[i+1, b]`), `lengths` the live keys per sequence.  16-bit storage, head dim 64 or 128.
"""
function paged_decode_attention!(O, Q, K_pages, V_pages; block_table, lengths, n_splits = nothing, scratch = nothing)
    Dq, H, B = size(Q)
    Dk, page_size, Hkv, n_pages = size(K_pages)
    Dv = size(V_pages, 1)
    @assert Dq == Dk
    @assert size(V_pages)[2:4] == (page_size, Hkv, n_pages)
    @assert size(O) == (Dv, H, B)
    @assert size(block_table, 2) == B
    @assert iszero(H % Hkv)
    max_pages = size(block_table, 1)
    eltype(block_table) === Int32 && eltype(lengths) === Int32 || throw(ArgumentError("block_table and lengths must be Int32"))
    if scratch === nothing
        n_splits === nothing && (n_splits = suggest_splits(page_size * max_pages, Hkv, B))
        scratch = allocate_scratchspace(decode_attention!, O, Q; n_splits)
    end
    (; O_partial, M_partial, L_partial, tickets) = scratch
    require_dense(O, Q, K_pages, V_pages, block_table, lengths, O_partial, M_partial, L_partial, tickets)
    check(ccall((:tylo_b200_decode_attention_paged, libtylo), Int32,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Ptr{Cvoid}),
        devptr(O), devptr(Q), devptr(K_pages), devptr(V_pages), devptr(block_table), devptr(lengths), devptr(O_partial),
        devptr(M_partial), devptr(L_partial), devptr(tickets), Int32(size(O_partial, 4)), Int32(page_size), Int32(max_pages),
        Int32(Dk), Int32(Dv), Int32(H), Int32(Hkv), Int32(B), tylo_dtype(eltype(Q)), current_stream()))
    return O
end

# ---- one sequence's keys sharded over the GPUs of a node (no counterpart in the reference) ------------

"""
    DecodeExchange(O; rank, world, share, timeout_us = 0)

Receive buffer of this process for sharded decode, mapped into every process of the node.
`share(handle::Vector{UInt8}) -> Vector{Vector{UInt8}}` is the host channel: it must return the
handles of all ranks in rank order (an MPI allgather, a file, a socket — 64 bytes per rank) and act
as a barrier.  The buffer lives until `close(ex)`.
"""
mutable struct DecodeExchange
    own::Ptr{Cvoid}
    peers::Vector{Ptr{Cvoid}}
    opened::Vector{Ptr{Cvoid}}
    rank::Int32
    world::Int32
    timeout_us::Int64
end

function DecodeExchange(O; rank::Integer, world::Integer, share, timeout_us::Integer = 0)
    Dv, H, B = size(O)
    nbytes = ccall((:tylo_b200_decode_exchange_bytes, libtylo), Int64, (Int32, Int32, Int32, Int32), world, Dv, H, B)
    nbytes > 0 || throw(ArgumentError("decode exchange: unsupported extents (world=$world, Dv=$Dv)"))
    own = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:tylo_b200_peer_alloc, libtylo), Int32, (Ptr{Ptr{Cvoid}}, Int64), own, nbytes))
    hb = ccall((:tylo_b200_peer_handle_bytes, libtylo), Int32, ())
    handle = zeros(UInt8, hb)
    check(ccall((:tylo_b200_peer_export, libtylo), Int32, (Ptr{Cvoid}, Ptr{UInt8}), own[], handle))
    handles = world > 1 ? share(handle) : [handle]
    peers = Vector{Ptr{Cvoid}}(undef, world); opened = Ptr{Cvoid}[]
    for r in 0:world-1
        if r == rank
            peers[r + 1] = own[]
        else
            p = Ref{Ptr{Cvoid}}(C_NULL)
            check(ccall((:tylo_b200_peer_open, libtylo), Int32, (Ptr{Ptr{Cvoid}}, Ptr{UInt8}), p, handles[r + 1]))
            peers[r + 1] = p[]; push!(opened, p[])
        end
    end
    return DecodeExchange(own[], peers, opened, Int32(rank), Int32(world), Int64(timeout_us))
end

function Base.close(ex::DecodeExchange)
    foreach(p -> ccall((:tylo_b200_peer_close, libtylo), Int32, (Ptr{Cvoid},), p), ex.opened)
    empty!(ex.opened)
    ex.own == C_NULL || ccall((:tylo_b200_peer_free, libtylo), Int32, (Ptr{Cvoid},), ex.own)
    ex.own = C_NULL
    return nothing
end

"""
    sharded_decode_attention!(O, Q, K_local, V_local; lengths_local, exchange, scratch, one_launch = false) -> O

`decode_attention!` when this process holds only a key range of every sequence.  Default: the split kernel
on the local keys, then the exchange kernel (placed while the splits still run), which merges the local
splits, pushes the merged records to every peer over NVLink, waits (bounded) for theirs and writes the final
`O` on every rank.  `one_launch = true` lets the split kernel's last block per (kv head, batch) do the merge
and the exchange itself (one launch; measured slower at 2 and 8 GPUs).  All ranks call it in the same order.
"""
function sharded_decode_attention!(O, Q, K, V; lengths_local, exchange::DecodeExchange, scratch, one_launch = false)
    Dk, Sk, Hkv, B = size(K)
    Dv, H, _ = size(O)
    (; O_partial, M_partial, L_partial) = scratch
    tickets = one_launch ? get(scratch, :tickets, nothing) : nothing      # without tickets the library takes two launches
    ns = size(O_partial, 4)
    require_dense(O, Q, K, V, lengths_local, O_partial, M_partial, L_partial, tickets)
    check(ccall((:tylo_b200_decode_attention_sharded, libtylo), Int32,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int32, Ptr{Ptr{Cvoid}}, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int32, Int64, Ptr{Cvoid}),
        devptr(O), devptr(Q), devptr(K), devptr(V), devptr(lengths_local), devptr(O_partial), devptr(M_partial),
        devptr(L_partial), devptr(tickets), Int32(ns), exchange.peers, exchange.rank, exchange.world, Int32(Dk),
        Int32(Dv), Int32(Sk), Int32(H), Int32(Hkv), Int32(B), tylo_dtype(eltype(Q)), exchange.timeout_us,
        current_stream()))
    return O
end

"Synchronises; throws if a peer's record did not arrive within the time limit in an earlier call."
function exchange_status(ex::DecodeExchange)
    code = Ref{Int32}(0)
    check(ccall((:tylo_b200_decode_exchange_status, libtylo), Int32, (Ptr{Cvoid}, Ptr{Int32}), ex.own, code))
    return Int(code[])
end
