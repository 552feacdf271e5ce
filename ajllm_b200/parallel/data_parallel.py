"""Replicated data parallelism on top of :class:`~ajllm_b200.training.optim.FlatAdamW`.

Each data-parallel rank sees different batches; because all parameters of a class sit contiguously in
the flat fp32 gradient buffer, the gradient reduction is one all-reduce per class instead of one per
tensor (the reference averages its replicated tensors one collective at a time,
``ajllm/training/distributed.py:351-366``). Losses are formed as ``local_mean / dp`` so every reduction
is a plain sum.
"""

from __future__ import annotations


def optimizer_classes(mesh, tp=None, cp=None) -> list[dict]:
    """Parameter classes for the flat optimizer under (tensor x data) parallelism. With context parallelism (``cp``,
    which then occupies the mesh's innermost axis instead of ``tp``) every parameter is replicated over the group and
    its gradient, computed from that rank's tokens only, is summed over it."""
    dp_group = mesh.dp.group if mesh.dp_size > 1 else None
    if cp is not None and cp.size > 1:
        return [{"name": "replicated", "match": lambda n, p: True,
                 "reduce_groups": [g for g in (cp.group, dp_group) if g is not None], "norm_groups": []}]

    def tp_sharded(name: str, p) -> bool:
        return tp is not None and tp.size > 1 and any(
            name.endswith(s) for s in ("attention.qkv_proj", "attention.output_proj", "feed_forward.w13",
                                       "feed_forward.w2", "feed_forward.w1"))

    def expert(name: str, p) -> bool:
        return ".experts." in name and mesh.ep_size > 1

    classes = [
        {"name": "experts", "match": expert,
         "reduce_groups": [mesh.ep_replica.group] if mesh.ep_replica.size > 1 else [],
         "norm_groups": [g for g in (mesh.ep.group, mesh.ep_replica.group if mesh.ep_replica.size > 1 else None) if g is not None]},
        {"name": "tp_sharded", "match": tp_sharded, "reduce_groups": [dp_group] if dp_group else [],
         "norm_groups": [tp.group] if (tp is not None and tp.size > 1) else []},
        {"name": "replicated", "match": lambda n, p: True,
         "reduce_groups": [g for g in ((tp.group if (tp is not None and tp.size > 1) else None), dp_group) if g is not None],
         "norm_groups": []},
    ]
    return classes
