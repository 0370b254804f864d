"""The plan of an online run: every rank derives the same packed rows from the dataset, and a trainer's ring
batch built from a packed row equals the batch the file path collates for the same dataset rows."""

import torch

from speculators_b200.models.eagle3.data import shift_batch
from speculators_b200.train.data import ArrowDataset, CollateFn
from speculators_b200.train.distributed_batch_sampler import MultipackDistributedBatchSamplerV2
from speculators_b200.train.online_data import OnlineBatchPlan
from speculators_b200.train.ring_loader import batch_from_ring_sample

H, LAYERS = 8, 4


def _dataset(root, n=14, seed=0):
    from datasets import Dataset
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(seed)
    rows = []
    for _ in range(n):
        L = int(torch.randint(6, 30, (1,), generator=g))
        rows.append({"input_ids": torch.randint(0, 90, (L,), generator=g).tolist(), "loss_mask": [0] * 2 + [1] * (L - 2), "seq_len": L})
    Dataset.from_list(rows).save_to_disk(str(root))
    (root / "hidden_states").mkdir()
    stored = []
    for i, r in enumerate(rows):
        hs = torch.randn(r["seq_len"], LAYERS, H, generator=g).to(torch.bfloat16)
        stored.append(hs)
        save_file({"hidden_states": hs, "token_ids": torch.tensor(r["input_ids"])}, str(root / "hidden_states" / f"hs_{i}.safetensors"))
    return rows, stored


def test_plan_rows_follow_the_multipack_sampler_and_match_the_file_path(tmp_path):
    rows, stored = _dataset(tmp_path / "ds")
    seq_len, n_trainer = 48, 2
    plan = OnlineBatchPlan(tmp_path / "ds", seq_len, n_trainer, seed=3)
    dataset = ArrowDataset(seq_len, tmp_path / "ds", on_missing="raise")
    collate = CollateFn(seq_len, H, LAYERS - 1, torch.bfloat16, preprocess=shift_batch)
    for epoch in (0, 1):
        plan.set_epoch(epoch)
        for ti in range(n_trainer):
            sampler = MultipackDistributedBatchSamplerV2(seq_len, [r["seq_len"] for r in rows], n_trainer, ti, seed=3)
            sampler.set_epoch(epoch)
            batches = [list(map(int, b)) for b in sampler]
            assert plan.steps_per_epoch <= len(batches)
            for step in range(plan.steps_per_epoch):
                row = plan.row(step, ti)
                want_ids = torch.cat([torch.tensor(rows[i]["input_ids"]) for i in batches[step]])[:seq_len]
                assert torch.equal(row["input_ids"], want_ids) and sum(row["lengths"]) == row["input_ids"].numel() <= seq_len
                assert row["position_ids"][0] == 0 and row["document_ids"].max() == len(row["lengths"]) - 1
                # what the verifier would push for this row (the documents' stored states, packed), seen from the trainer
                packed = torch.cat([stored[i] for i in batches[step]])[:seq_len].flatten(1)
                got = batch_from_ring_sample({"hidden_states": packed, "token_ids": row["input_ids"]}, H, seq_len, loss_mask=row["loss_mask"],
                                             lengths=row["lengths"])
                want = collate([dataset[i] for i in batches[step]])
                for key in want:
                    assert torch.equal(got[key].to(want[key].dtype), want[key]), (epoch, ti, step, key)
    assert plan.steps_per_epoch >= 2
