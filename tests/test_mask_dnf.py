"""CPU: the disjunctive normal form the host layer passes to the library keeps the meaning of the mask
tree (AndMask / OrMask / prefix_lm, mods.jl:151-178), checked pair by pair with the host evaluator."""
import itertools
import random

import torch


def _trees(t):
    docs = torch.tensor([0, 0, 1, 1, 1, 2, 2, 3, 3, 3, 3, 4], dtype=torch.int32)
    atoms = [t.CausalMask(), t.SlidingWindowMask(2), t.SlidingWindowMask(5), t.PrefixMask(3), t.PrefixMask(7),
             t.DocumentMask(docs), t.FullMask()]
    rnd = random.Random(3)

    def grow(depth):
        if depth == 0 or rnd.random() < 0.3:
            return rnd.choice(atoms)
        a, b = grow(depth - 1), grow(depth - 1)
        return (a & b) if rnd.random() < 0.5 else (a | b)

    return [grow(3) for _ in range(60)] + [t.prefix_lm(4), t.prefix_lm(4) & t.SlidingWindowMask(5),
                                           t.CausalMask() | (t.PrefixMask(3) & t.DocumentMask(docs))]


def test_dnf_keeps_the_meaning(tylo):
    t = tylo
    for tree in _trees(t):
        clauses = t._mask_clauses(tree)
        for q, kv in itertools.product(range(12), range(12)):
            want = bool(t.hmask(tree, q, kv))
            got = any(all(bool(term(1, 1, q, kv)) for term in clause) for clause in clauses)
            assert got == want, (tree, q, kv)


def test_prefix_lm_stays_one_term(tylo):
    t = tylo
    assert len(t._mask_clauses(t.prefix_lm(5))) == 1
    assert len(t._mask_clauses(t.prefix_lm(5) & t.SlidingWindowMask(3))) == 1
    assert len(t._mask_clauses((t.CausalMask() & t.SlidingWindowMask(3)) | t.PrefixMask(2))) == 2
