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


def test_serve_and_training_loader_walk_the_plan_in_step(tmp_path):
    """The two halves of an in-job online run, joined through a stand-in ring on the CPU: what the verifier side
    pushes for (epoch, step, trainer) is what the trainer side's loader pairs with that step's mask and lengths."""
    from types import SimpleNamespace

    from speculators_b200.train.online import OnlineSplit

    rows, stored = _dataset(tmp_path / "ds")
    seq_len = 48
    plan = OnlineBatchPlan(tmp_path / "ds", seq_len, 1, seed=5)
    pushed = []

    class FakeVerifier:
        comm = None

        def forward(self, ids, aux_layers, document_ids=None, position_ids=None):
            # "hidden states" that encode the token and its place, so that a mix-up of rows shows
            base = torch.stack([ids.float(), document_ids.float(), position_ids.float(), torch.ones_like(ids).float()], dim=-1)
            return {"hidden_states": base.repeat(1, 2 * (LAYERS - 1)).to(torch.bfloat16), "verifier_last_hidden_states": (base * 2).repeat(1, 2).to(torch.bfloat16)}

    class FakeWriter:
        def push(self, seq, payload, ids, timeout_s, check):
            pushed.append((seq, payload.clone(), ids.clone()))

        def check_status(self):
            pass

    class FakeRing:
        def pop(self, seq, timeout_s):
            s, payload, ids = pushed[seq - 1]
            assert s == seq
            return {"hidden_states": payload, "token_ids": ids.long()}

    def make(is_verifier):
        split = object.__new__(OnlineSplit)
        split.__dict__.update(plan=plan, transform=None, topo=SimpleNamespace(n_trainer=1, is_verifier=is_verifier, trainer_index=0),
                              device=torch.device("cpu"), aux_layers=[0, 1, 2], hidden=H, seq_len=seq_len, timeout_s=1.0, writers={0: FakeWriter()},
                              verifier=FakeVerifier(), ring=FakeRing(), _seq=0)
        return split

    served = make(True).serve(first_epoch=0, num_epochs=2)
    per_epoch = []
    for epoch in (0, 1):
        plan.set_epoch(epoch)
        per_epoch.append(plan.steps_per_epoch)
    assert served == sum(per_epoch) == len(pushed)

    loader = make(False).training_loader()
    n = 0
    for epoch in (0, 1):
        loader.batch_sampler.set_epoch(epoch)
        assert len(loader) == per_epoch[epoch]
        for step, batch in enumerate(loader):
            row = plan.row(step, 0)
            keep = int((batch["document_ids"][0] != -1).sum())
            assert keep == sum(max(0, L - 1) for L in row["lengths"])
            # the token ids of the batch are the row's ids shifted inside every document
            want_ids = torch.cat([row["input_ids"][s + 1 : s + L] for s, L in zip([sum(row["lengths"][:i]) for i in range(len(row["lengths"]))], row["lengths"])])
            assert torch.equal(batch["input_ids"][0, :keep], want_ids)
            # hidden state of position t belongs to token t (first channel carries the token id)
            want_prev = torch.cat([row["input_ids"][s : s + L - 1] for s, L in zip([sum(row["lengths"][:i]) for i in range(len(row["lengths"]))], row["lengths"])])
            assert torch.equal(batch["hidden_states"][0, :keep, 0].long(), want_prev)
            assert torch.equal(batch["loss_mask"][0, :keep], torch.cat([row["loss_mask"][s + 1 : s + L] for s, L in zip([sum(row["lengths"][:i]) for i in range(len(row["lengths"]))], row["lengths"])]))
            n += 1
    assert n == served
    # a step budget ends the verifier side early
    pushed.clear()
    assert make(True).serve(first_epoch=0, num_epochs=2, max_steps=3) == 3 and len(pushed) == 3
