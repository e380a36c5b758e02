"""Unit-level contracts of the distributed stack that need no process group.

Behaviour pinned here follows the reference's suites
(distributed/tests/test_optim_shard.py, test_tensor_parallel.py:150-163,
test_train.py:49-71): the sharded optimizer validates its parameter list and guards a
restored shard by rank / world / layout, every rank derives the same ownership table even
when it owns nothing, model surgery checks all layers before it changes any, the runner
refuses to write into an existing directory, and tensor-parallel ranks all see the whole
global batch.
"""

import pytest
import torch
import torch.distributed as dist

from systems_for_llms_b200.config import load_config
from systems_for_llms_b200.models.transformer import TransformerLM
from systems_for_llms_b200.parallel import tensor_parallel as tp_module
from systems_for_llms_b200.parallel.optim_shard import ShardedAdamW, assign_owners
from systems_for_llms_b200.parallel.train import run, validate_layout


class FakeGroup:
    """Stands in for an initialised process group of ``world`` ranks seen from ``rank``."""

    def __init__(self, monkeypatch, world: int):
        self.world, self.rank = world, 0
        monkeypatch.setattr(dist, "is_initialized", lambda: True)
        monkeypatch.setattr(dist, "get_world_size", lambda group=None: self.world)
        monkeypatch.setattr(dist, "get_rank", lambda group=None: self.rank)
        monkeypatch.setattr(dist, "all_gather_object", self._gather)

    def _gather(self, out, value, group=None):
        out[:] = [value] * self.world      # every rank reports the same shapes


def test_parameter_list_is_validated():
    weight = torch.nn.Parameter(torch.zeros(3))
    with pytest.raises(ValueError, match="at least one"):
        ShardedAdamW(())
    with pytest.raises(ValueError, match="Duplicate"):
        ShardedAdamW([weight, torch.nn.Parameter(torch.zeros(1)), weight])


def test_shard_state_restores_only_into_the_same_rank_and_layout():
    weight = torch.nn.Parameter(torch.tensor([0.25, -1.5, 3.0], dtype=torch.float64))
    first = ShardedAdamW([weight], lr=0.02, weight_decay=0.0)
    weight.grad = torch.tensor([1.0, -0.5, 0.25], dtype=torch.float64)
    first.step()
    assert first.local_state_bytes() >= 2 * weight.numel() * 8     # two moments, fp64
    saved = first.state_dict()

    first.zero_grad(set_to_none=False)
    assert weight.grad is not None and not weight.grad.any()
    first.zero_grad()
    assert weight.grad is None

    second = ShardedAdamW([weight], lr=0.02, weight_decay=0.0)
    second.load_state_dict(saved)
    assert second.local_state_bytes() == first.local_state_bytes()
    for field, wrong in (("rank", 1), ("world_size", 2)):
        tampered = {**saved, "sharding": {**saved["sharding"], field: wrong}}
        with pytest.raises(ValueError, match="does not match"):
            second.load_state_dict(tampered)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_every_rank_derives_the_same_owner_table(monkeypatch, world):
    group = FakeGroup(monkeypatch, world)
    sizes = (11, 6, 6, 2)
    tables, owned = [], []
    for rank in range(world):
        group.rank = rank
        optimizer = ShardedAdamW([torch.nn.Parameter(torch.zeros(n)) for n in sizes])
        meta = optimizer.ownership_metadata()
        tables.append(meta["owners"])
        owned.append(meta["owned_parameter_indices"])
        assert sum(len(g["params"]) for g in optimizer.param_groups) == len(owned[-1])
        assert optimizer.local_state_bytes() == 0          # no state before the first step
    assert all(table == tables[0] for table in tables)
    assert sorted(i for mine in owned for i in mine) == list(range(len(sizes)))
    assert tables[0] == assign_owners(list(sizes), world)[0]
    if world > len(sizes):
        assert any(not mine for mine in owned)              # some ranks own nothing


def small_model():
    return TransformerLM(vocab_size=40, context_length=8, d_model=16, num_layers=3, num_heads=4,
                         d_ff=24, rope_theta=10000.0, attention_backend="eager")


def test_surgery_needs_a_process_group():
    with pytest.raises(RuntimeError, match="initialized process group"):
        tp_module.parallelize_model(small_model())


def test_surgery_checks_all_layers_before_changing_one(monkeypatch):
    monkeypatch.setattr(tp_module, "_world", lambda group: (3, 1))     # 4 heads over 3 ranks
    model = small_model()
    before = [(layer.attn, layer.ffn) for layer in model.layers]
    with pytest.raises(ValueError, match="head count"):
        tp_module.parallelize_model(model)
    assert all(layer.attn is attn and layer.ffn is ffn
               for layer, (attn, ffn) in zip(model.layers, before))


def test_runner_refuses_an_existing_output_directory(tmp_path):
    target = tmp_path / "taken"
    target.mkdir()
    (target / "summary.json").write_text("kept\n")
    with pytest.raises(FileExistsError):
        run(load_config("configs/smoke.json"), target, warmup_steps=1)
    assert (target / "summary.json").read_text() == "kept\n"
    assert sorted(p.name for p in target.iterdir()) == ["summary.json"]


def test_microbatches_per_rank_by_mode():
    # data-parallel ranks split the global batch, tensor-parallel ranks all see it
    assert validate_layout("ddp", 4, 16, 2, "last") == 2
    assert validate_layout("zero1", 2, 8, 1, "last") == 4
    assert validate_layout("tp", 2, 8, 1, "last") == 8
    assert validate_layout("tp", 8, 8, 2, "last") == 4
