"""SPMD inference rules: input re-sharding and output layouts per operator family, on dims_mappings only (no process
group).  Cases follow the reference's rule tests (test/auto_parallel/spmd_rules/test_*_rule.py) on a 2 x 3 mesh."""
import pytest

from paddle_b200.distributed.auto_parallel.spmd_rules import get_phi_spmd_rule, has_rule, rule_names, spec

MESH = [2, 3]


def fwd(name, *args, **kw):
    ins, outs = get_phi_spmd_rule(name).infer_forward(*args, **kw)
    return ins, outs


def dm(specs):
    return [s.dims_mapping if not isinstance(s, list) else [t.dims_mapping for t in s] for s in specs]


def test_registry_covers_the_reference_rule_files():
    for n in ("add_n", "argmax", "c_embedding", "c_softmax_with_cross_entropy", "cast", "clip", "concat", "conv2d", "cross_entropy_with_softmax",
              "cumsum", "default_data_parallel", "dropout", "elementwise", "embedding", "expand_as", "flash_attention", "flatten", "full_like",
              "fused_dropout_add", "fused_linear_param_grad_add", "fused_rope", "gather", "gather_nd", "layer_norm", "logsumexp", "matmul",
              "moe_combine", "moe_gate_dispatch", "nonzero", "numel", "one_hot", "optimizer", "p_norm", "pad", "pow", "reduction", "replicated",
              "reshape", "rms_norm", "scale", "scatter", "slice", "softmax", "split", "squared_l2_norm", "squeeze", "stack", "swiglu", "tile",
              "transpose", "triu", "unbind", "unsqueeze", "where", "amp_ops"):
        assert has_rule(n), n
    assert len(rule_names()) > 150
    with pytest.raises(KeyError):
        get_phi_spmd_rule("no_such_rule")


def test_matmul_rule():
    x, y = spec([64, 32], [1, 0]), spec([32, 48], [-1, -1])
    ins, outs = fwd("matmul", x, y, False, False)
    assert dm(ins) == [[1, 0], [0, -1]] and outs[0].dims_mapping == [1, -1] and outs[0].partial_dims == {0}
    ins, outs = fwd("matmul", spec([64, 32], [1, -1]), y, False, False)
    assert dm(ins) == [[1, -1], [-1, -1]] and outs[0].dims_mapping == [1, -1] and not outs[0].is_partial()
    ins, outs = fwd("matmul", spec([64, 32]), spec([32, 48], [-1, 0]))
    assert outs[0].dims_mapping == [-1, 0] and not outs[0].is_partial()
    ins, outs = fwd("matmul", spec([64, 32]), spec([32, 48], [1, 0]))
    assert dm(ins) == [[-1, 1], [1, 0]] and outs[0].dims_mapping == [-1, 0] and outs[0].partial_dims == {1}
    ins, outs = fwd("matmul", spec([512, 48, 64, 32], [1, -1, -1, 0]), spec([32, 48]))
    assert dm(ins) == [[1, -1, -1, 0], [0, -1]] and outs[0].dims_mapping == [1, -1, -1, -1] and outs[0].partial_dims == {0}
    # a mesh axis cannot split both m and n: the later letter gives way
    ins, outs = fwd("matmul", spec([64, 32], [0, -1]), spec([32, 48], [-1, 0]))
    assert dm(ins) == [[0, -1], [-1, -1]] and outs[0].dims_mapping == [0, -1]
    # transposes
    ins, outs = fwd("matmul", spec([32, 64], [-1, 0]), spec([48, 32], [1, -1]), True, True)
    assert outs[0].shape == [64, 48] and outs[0].dims_mapping == [0, 1]
    # batched broadcast: [b, m, k] x [k, n]; and the backward inference from the output layout
    ins, outs = fwd("matmul", spec([8, 64, 32], [0, -1, -1]), spec([32, 48], [-1, 1]))
    assert outs[0].dims_mapping == [0, -1, 1]
    ins, _ = get_phi_spmd_rule("matmul").infer_backward(spec([8, 64, 32]), spec([32, 48]), spec([8, 64, 48], [0, -1, 1]))
    assert dm(ins) == [[0, -1, -1], [-1, 1]]


def test_elementwise_and_reduction_rules():
    ins, outs = fwd("add", spec([64, 36], [0, -1]), spec([36], [1]))
    assert dm(ins) == [[0, 1], [1]] and outs[0].dims_mapping == [0, 1]
    ins, outs = fwd("multiply", spec([64, 1, 36], [0, -1, -1]), spec([48, 36], [1, -1]))
    assert outs[0].shape == [64, 48, 36] and outs[0].dims_mapping == [0, 1, -1] and dm(ins) == [[0, -1, -1], [1, -1]]
    ins, outs = fwd("where", spec([8, 16], [0, -1]), spec([8, 16]), spec([16], [1]))
    assert outs[0].dims_mapping == [0, 1] and dm(ins) == [[0, 1], [0, 1], [1]]
    ins, _ = get_phi_spmd_rule("add").infer_backward(spec([64, 36]), spec([36]), spec([64, 36], [0, 1]))
    assert dm(ins) == [[0, 1], [1]]
    ins, outs = fwd("sum", spec([64, 32], [0, -1]), [0], False)
    assert outs[0].dims_mapping == [-1] and outs[0].partial_dims == {0} and dm(ins) == [[0, -1]]
    ins, outs = fwd("max", spec([64, 32], [0, 1]), [1], True)
    assert outs[0].shape == [64, 1] and outs[0].dims_mapping == [0, -1] and outs[0].partial_dims == {1}
    ins, outs = fwd("sum", spec([4, 8, 16], [-1, 0, 1]), [0, 2], False)
    assert outs[0].dims_mapping == [0] and outs[0].partial_dims == {1}
    ins, outs = fwd("logsumexp", spec([64, 32], [0, 1]), [1], False)
    assert dm(ins) == [[0, -1]] and outs[0].dims_mapping == [0] and not outs[0].is_partial()
    ins, outs = fwd("squared_l2_norm", spec([64, 32], [0, 1]))
    assert outs[0].shape == [] and outs[0].partial_dims == {0, 1}
    ins, outs = fwd("argmax", spec([64, 32], [0, 1]), 1, False)
    assert dm(ins) == [[0, -1]] and outs[0].dims_mapping == [0]
    ins, outs = fwd("cumsum", spec([64, 32], [0, 1]), 1)
    assert dm(ins) == [[0, -1]] and outs[0].dims_mapping == [0, -1]
    ins, outs = fwd("p_norm", spec([64, 32], [0, 1]), 2.0, 0, 1e-12, False, False)
    assert dm(ins) == [[-1, 1]] and outs[0].dims_mapping == [1]


def test_norm_softmax_embedding_and_loss_rules():
    ins, outs = fwd("softmax", spec([16, 32, 48], [0, -1, 1]), -1)
    assert dm(ins) == [[0, -1, -1]] and outs[0].dims_mapping == [0, -1, -1]
    ins, outs = fwd("layer_norm", spec([64, 32, 1024], [1, -1, 0]), spec([1024], [0]), spec([1024]), 1e-5, 2)
    assert dm(ins) == [[1, -1, -1], [-1], [-1]] and dm(outs) == [[1, -1, -1], [1, -1], [1, -1]]
    ins, outs = fwd("layer_norm", spec([64, 32, 1024], [0, 1, -1]), spec([32 * 1024]), spec([32 * 1024]), 1e-5, 1)
    assert dm(ins)[0] == [0, -1, -1] and dm(outs) == [[0, -1, -1], [0], [0]]
    ins, outs = fwd("rms_norm", spec([8, 128, 4096], [0, 1, -1]), spec([4096]))
    assert dm(outs) == [[0, 1, -1], [0, 1]]
    # embedding: row-parallel table -> partial; column-parallel -> last dim split
    ins, outs = fwd("embedding", spec([4, 1024], [0, -1]), spec([512, 768], [1, -1]))
    assert outs[0].shape == [4, 1024, 768] and outs[0].dims_mapping == [0, -1, -1] and outs[0].partial_dims == {1}
    ins, outs = fwd("embedding", spec([4, 1024], [0, -1]), spec([512, 768], [-1, 1]))
    assert outs[0].dims_mapping == [0, -1, 1] and not outs[0].is_partial()
    ins, outs = fwd("embedding", spec([4, 1024], [0, -1]), spec([512, 768], [0, -1]))      # the axis is taken by the batch
    assert dm(ins) == [[0, -1], [-1, -1]]
    # cross entropy: class dim may stay split (vocab parallel); loss has size 1 there
    ins, outs = fwd("cross_entropy_with_softmax", spec([32, 48], [0, 1]), spec([32, 1], [-1, -1]), False, True, True, -100, -1)
    assert dm(ins) == [[0, 1], [0, -1]] and dm(outs) == [[0, 1], [0, -1]] and outs[1].shape == [32, 1]
    ins, outs = fwd("cross_entropy_with_softmax", spec([32, 48], [-1, 0]), spec([32, 48], [1, -1]), True, True, True, -100, 1)
    assert dm(ins) == [[1, 0], [1, 0]] and dm(outs) == [[1, 0], [1, -1]]


def test_layout_rules():
    ins, outs = fwd("transpose", spec([64, 48, 36, 24], [0, 1, -1, -1]), [1, 2, 3, 0])
    assert outs[0].shape == [48, 36, 24, 64] and outs[0].dims_mapping == [1, -1, -1, 0]
    x = lambda m: spec([6, 12, 48, 24], m)
    cases = [([0, -1, 1, -1], [1, 72, 48, 4, 6], [0, -1, 1, -1], [-1, 0, 1, -1, -1]),
             ([-1, 0, -1, 1], [1, 72, 48, 4, 6], [-1, -1, -1, -1], [-1, -1, -1, -1, -1]),
             ([1, -1, -1, 0], [1, 72, 48, 4, 6], [1, -1, -1, 0], [-1, 1, -1, 0, -1]),
             ([0, 1, -1, -1], [3, 24, 6, 8, 24], [-1, -1, -1, -1], [-1, -1, -1, -1, -1]),
             ([1, -1, -1, 0], [3, 24, 6, 8, 24], [1, -1, -1, 0], [1, -1, -1, -1, 0]),
             ([-1, -1, 0, 1], [3, 24, 6, -1, 24], [-1, -1, 0, 1], [-1, -1, 0, -1, 1]),
             ([1, -1, -1, 0], [1, 72, 0, 4, 6], [1, -1, -1, 0], [-1, 1, -1, 0, -1]),
             ([0, -1, 1, -1], [72, 3, 16, 24], [0, -1, 1, -1], [0, 1, -1, -1]),
             ([1, -1, 0, -1], [72, 3, 16, 24], [1, -1, -1, -1], [1, -1, -1, -1])]
    for src, shape, want_in, want_out in cases:
        ins, outs = fwd("reshape", x(src), shape, mesh_shape=MESH)
        assert (ins[0].dims_mapping, outs[0].dims_mapping) == (want_in, want_out), (src, shape)
    ins, outs = fwd("reshape", spec([1, 72, 48, 4, 6], [-1, 1, -1, 0, -1]), [6, 12, 48, 24], mesh_shape=MESH)
    assert outs[0].dims_mapping == [1, -1, -1, 0]
    ins, outs = fwd("reshape", spec([8, 1024, 3072], [0, 1, -1]), [0, 0, -1, 192], mesh_shape=MESH)
    assert outs[0].shape == [8, 1024, 16, 192] and outs[0].dims_mapping == [0, 1, -1, -1]
    ins, outs = fwd("squeeze", spec([1, 8, 1, 16], [-1, 0, -1, 1]), [0, 2])
    assert outs[0].shape == [8, 16] and outs[0].dims_mapping == [0, 1]
    ins, outs = fwd("unsqueeze", spec([8, 16], [0, 1]), [0, -1])
    assert outs[0].shape == [1, 8, 16, 1] and outs[0].dims_mapping == [-1, 0, 1, -1]
    ins, outs = fwd("concat", [spec([16, 16, 16], [-1, 0, 1]), spec([4, 16, 16], [0, -1, -1])], 0)
    assert dm(ins) == [[[-1, 0, 1], [-1, 0, 1]]] and outs[0].shape == [20, 16, 16] and outs[0].dims_mapping == [-1, 0, 1]
    ins, outs = fwd("stack", [spec([8, 16], [0, -1]), spec([8, 16], [-1, 1])], 1)
    assert outs[0].shape == [8, 2, 16] and outs[0].dims_mapping == [0, -1, 1] and dm(ins) == [[[0, 1], [0, 1]]]
    ins, outs = fwd("split", spec([64, 48, 36], [0, 1, -1]), [16, 16, -1], 1)
    assert dm(ins) == [[0, -1, -1]] and [o.shape for o in outs[0]] == [[64, 16, 36]] * 3 and dm(outs) == [[[0, -1, -1]] * 3]
    ins, outs = fwd("split_with_num", spec([64, 48, 36], [0, -1, 1]), 3, 1)
    assert dm(outs) == [[[0, -1, 1]] * 3]
    ins, outs = fwd("unbind", spec([3, 8, 16], [0, 1, -1]), 0)
    assert dm(ins) == [[-1, 1, -1]] and len(outs[0]) == 3 and outs[0][0].dims_mapping == [1, -1]
    ins, outs = fwd("slice", spec([64, 48, 36], [0, 1, -1]), [1, 2], [4, 0], [20, 18], None, [])
    assert dm(ins) == [[0, -1, -1]] and outs[0].shape == [64, 16, 18] and outs[0].dims_mapping == [0, -1, -1]
    ins, outs = fwd("slice", spec([64, 48], [0, 1]), [1], [3], [4], None, [1])
    assert outs[0].shape == [64] and outs[0].dims_mapping == [0]
    ins, outs = fwd("tile", spec([8, 16], [0, 1]), [2, 1, 3])
    assert outs[0].shape == [2, 8, 48] and dm(ins) == [[0, -1]] and outs[0].dims_mapping == [-1, 0, -1]
    ins, outs = fwd("expand_as", spec([1, 16], [-1, 1]), None, [8, 4, 16])
    assert outs[0].dims_mapping == [-1, -1, 1]
    ins, outs = fwd("pad", spec([8, 16, 32], [0, 1, -1]), [0, 0, 1, 1, 0, 0])
    assert dm(ins) == [[0, -1, -1]] and outs[0].shape == [8, 18, 32]
    ins, outs = fwd("triu", spec([4, 16, 16], [0, 1, -1]), 0)
    assert dm(ins) == [[0, -1, -1]]
    ins, outs = fwd("one_hot", spec([8, 16], [0, 1]), 10)
    assert outs[0].shape == [8, 16, 10] and outs[0].dims_mapping == [0, 1, -1]
    ins, outs = fwd("flatten", spec([8, 16, 32], [0, -1, -1]), [8 * 16, 32], mesh_shape=MESH)
    assert outs[0].dims_mapping == [0, -1]


def test_indexing_and_block_rules():
    ins, outs = fwd("gather", spec([64, 32], [0, 1]), spec([16], [-1]), 0)
    assert dm(ins) == [[-1, 1], [-1]] and outs[0].shape == [16, 32] and outs[0].dims_mapping == [-1, 1]
    ins, outs = fwd("gather", spec([64, 32], [-1, 1]), spec([16], [0]), 0)
    assert outs[0].dims_mapping == [0, 1]
    ins, outs = fwd("gather_nd", spec([10, 20, 30], [0, -1, 1]), spec([4, 5, 2], [-1, 0, -1]))
    assert dm(ins) == [[-1, -1, 1], [-1, 0, -1]] and outs[0].shape == [4, 5, 30] and outs[0].dims_mapping == [-1, 0, 1]
    ins, outs = fwd("scatter", spec([64, 32], [0, 1]), spec([16], [0]), spec([16, 32], [-1, -1]))
    assert dm(ins) == [[-1, 1], [-1], [-1, 1]] and outs[0].dims_mapping == [-1, 1]
    q = spec([8, 1024, 32, 128], [0, 1, -1, -1])
    kv = spec([8, 1024, 32, 128], [0, -1, 1, -1])
    ins, outs = fwd("flash_attention", q, kv, kv, None, 0.0, True)
    assert dm(ins) == [[0, -1, 1, -1]] * 3 and dm(outs) == [[0, -1, 1, -1], [0, 1, -1]]
    ins, outs = fwd("flash_attention", spec([8, 1024, 32, 128], [0, -1, 1, -1]), spec([8, 1024, 8, 128]), spec([8, 1024, 8, 128]))
    assert dm(ins)[1] == [0, -1, 1, -1]                        # grouped-query heads follow q's head split
    ins, outs = fwd("fused_rope", spec([8, 1024, 32, 128], [0, 1, -1, -1]), spec([8, 1024, 32, 128], [0, -1, -1, 1]), None,
                    spec([1, 1024, 1, 128]), spec([1, 1024, 1, 128]))
    assert dm(ins) == [[0, 1, -1, -1], [0, 1, -1, -1], [-1, 1, -1, -1], [-1, 1, -1, -1]] and dm(outs) == [[0, 1, -1, -1]] * 2
    ins, outs = fwd("swiglu", spec([8, 128, 1024], [0, -1, 1]))
    assert dm(ins) == [[0, -1, -1]] and outs[0].shape == [8, 128, 512]
    ins, outs = fwd("swiglu", spec([8, 128, 512], [0, -1, 1]), spec([8, 128, 512]))
    assert outs[0].dims_mapping == [0, -1, 1]
    ins, outs = fwd("fused_linear_param_grad_add", spec([8, 128, 512], [0, -1, -1]), spec([8, 128, 1024], [0, -1, 1]))
    assert dm(outs) == [[-1, 1], [1]] and outs[0].partial_dims == {0}
    ins, outs = fwd("conv2d", spec([8, 64, 32, 32], [0, -1, 1, -1]), spec([128, 64, 3, 3], [1, -1, -1, -1]))
    assert dm(ins) == [[0, -1, -1, -1], [1, -1, -1, -1]] and outs[0].dims_mapping == [0, 1, -1, -1]
    ins, outs = fwd("conv2d", spec([8, 64, 32, 32], [-1, 0, -1, -1]), spec([128, 64, 3, 3]))
    assert dm(ins)[1] == [-1, 0, -1, -1] and outs[0].partial_dims == {0}
    ins, outs = fwd("optimizer", spec([512, 512], [-1, 0]), spec([512, 512], [-1, -1]), spec([512, 512]), spec([512, 512]), spec([1]))
    assert dm(ins) == [[-1, 0]] * 4 + [[-1]] and len(outs) == 4
    ins, outs = fwd("amp_ops", [spec([8, 8], [0, -1]), spec([8], [1])], spec([1]))
    assert outs[1].partial_dims == {0, 1}
    ins, outs = fwd("default_data_parallel", spec([16, 8], [-1, 1]), spec([16], [-1]))
    assert dm(ins) == [[0, -1], [0]]
    ins, outs = fwd("nonzero", spec([8, 8], [0, 1]))
    assert dm(ins) == [[-1, -1]] and outs == []
    ins, outs = fwd("add_n", [spec([8, 8], [0, -1]), spec([8, 8], [-1, 1])])
    assert dm(ins) == [[[0, 1], [0, 1]]] and outs[0].dims_mapping == [0, 1]
    ins, outs = fwd("moe_gate_dispatch", spec([1024, 512], [0, -1]), spec([1024, 8], [-1, 1]), 2, 256)
    assert dm(ins) == [[0, -1], [0, -1]] and outs[0].shape == [8, 256, 512] and outs[0].partial_dims == {0}
