"""``decompose``: rewrite the composite nodes of a recorded program into primitive nodes
(python/paddle/decomposition/decomp.py:194-232)."""
from __future__ import annotations

import torch
from torch.utils import _pytree as pytree

from ..static import graph as G
from .primitives import PRIMITIVES
from .register import get_decomp_rule


def _examples(program):
    """slot -> example tensor of the recording pass."""
    ex = {}
    for t in program._keep:
        s = program._slot_of_id.get(id(t))
        if s is not None:
            ex[s] = t
    ex.update(program._captured)
    return ex


def _remap(obj, mapping):
    return pytree.tree_map(lambda a: G._Ref(mapping.get(a.slot, a.slot)) if isinstance(a, G._Ref) else a, obj)


def decompose(program, src_vars=None, blacklist=frozenset(), whitelist=frozenset(), start_index=0, end_index=-1):
    """Replace, in place, every node of ``program`` (its global block, nodes ``[start_index, end_index)``) that has a
    registered rule by the primitive nodes the rule expands to.  ``blacklist``: operator names that stay composite;
    ``whitelist``: when non-empty, only these are decomposed.  The variables in ``src_vars`` keep their identity (a
    rule's results are bound to the slots of the node it replaces), and are returned, as the reference returns the
    replaced values.  Rules are traced on the example values of the recording pass."""
    if not isinstance(program, G.Program):
        raise TypeError(f"expected a static Program, got {type(program).__name__}")
    blacklist = {b.split(".", 1)[-1] for b in blacklist}
    whitelist = {w.split(".", 1)[-1] for w in whitelist}
    nodes = program._nodes
    end = len(nodes) if end_index in (-1, None) else end_index
    examples = _examples(program)
    was_enabled = G._S.enabled
    if not was_enabled:
        G.enable()
    out_nodes = []
    try:
        with G.program_guard(program):
            for idx, node in enumerate(nodes):
                name = node.type
                rule = get_decomp_rule(name) if start_index <= idx < end else None
                if rule is None or name in blacklist or (whitelist and name not in whitelist):
                    out_nodes.append(node)
                    continue
                try:
                    args = pytree.tree_map(lambda a: examples[a.slot] if isinstance(a, G._Ref) else a, node.args)
                    kwargs = pytree.tree_map(lambda a: examples[a.slot] if isinstance(a, G._Ref) else a, node.kwargs)
                except KeyError:
                    out_nodes.append(node)          # an input without an example value: leave the node alone
                    continue
                with program._sub_block() as sub:
                    out = rule(*args, **kwargs)
                leaves = [o for o in pytree.tree_leaves(out) if isinstance(o, torch.Tensor)]
                if len(leaves) != len(node.out_slots) or not sub:
                    out_nodes.append(node)          # the rule fell back to the composite call or produced other arity
                    continue
                mapping = {}
                for o, s in zip(leaves, node.out_slots):
                    new = program._slot_of_id.get(id(o))
                    if new is None:
                        mapping = None
                        break
                    mapping[new] = s
                if mapping is None:
                    out_nodes.append(node)
                    continue
                for n in sub:
                    n.args, n.kwargs = _remap(n.args, mapping), _remap(n.kwargs, mapping)
                    n.out_slots = [mapping.get(s, s) for s in n.out_slots]
                # later rules are traced on the ORIGINAL example values of their inputs (looked up by object identity,
                # which still resolves to the replaced node's slots), so nothing else has to be updated
                out_nodes.extend(sub)
    finally:
        if not was_enabled:
            G.disable()
    program._nodes[:] = out_nodes
    program._version += 1
    return list(src_vars) if src_vars is not None else None


def is_primitive_program(program, allow=()):
    """True when every node of the program is a primitive operator (or named in ``allow``)."""
    allow = set(allow)
    return all(n.type in PRIMITIVES or n.type in allow for n in program._nodes)
