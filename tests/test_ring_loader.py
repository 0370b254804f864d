"""The device-side batch builder of the NVLink ring path must give what the file path gives:
dataset split of the stored ``[seq, layers, H]`` states -> pairing shift -> packed collate."""

import torch

from speculators_b200.models.eagle3.data import shift_batch
from speculators_b200.train.data import CollateFn, split_hidden_state_layers
from speculators_b200.train.ring_loader import RingBatchLoader, batch_from_ring_sample


def _sample(rows, layers=4, H=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    stored = torch.randn(rows, layers, H, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 100, (rows,), generator=g)
    mask = torch.rand(rows, generator=g) > 0.4
    return stored, ids, mask


def _file_path_batch(stored, ids, mask, seq_len, H, layers):
    aux, last = split_hidden_state_layers(stored)
    rows = ids.shape[0]
    item = {"hidden_states": aux, "input_ids": ids, "verifier_last_hidden_states": last, "loss_mask": mask,
            "lengths": torch.tensor([rows]), "position_ids": torch.arange(rows)}
    return CollateFn(seq_len, H, layers - 1, torch.bfloat16, preprocess=shift_batch)([item])


def test_ring_sample_batch_equals_collated_file_sample():
    H, layers = 8, 4
    for rows, seq_len in ((20, 32), (33, 32), (40, 32), (2, 16)):
        stored, ids, mask = _sample(rows, layers, H, seed=rows)
        want = _file_path_batch(stored, ids, mask, seq_len, H, layers)
        got = batch_from_ring_sample({"hidden_states": stored.flatten(1), "token_ids": ids}, H, seq_len, loss_mask=mask)
        assert set(got) == set(want)
        for key in want:
            assert got[key].shape == want[key].shape, key
            assert torch.equal(got[key].to(want[key].dtype), want[key]), (rows, seq_len, key)


def test_ring_batch_loader_pops_in_sequence():
    class FakeRing:
        def __init__(self):
            self.asked = []

        def pop(self, seq, timeout_s):
            self.asked.append(seq)
            stored, ids, _ = _sample(10, seed=seq)
            return {"hidden_states": stored.flatten(1), "token_ids": ids}

    ring = FakeRing()
    loader = RingBatchLoader(ring, num_steps=3, hidden_size=8, seq_len=16, first_seq=5)
    batches = list(loader)
    assert ring.asked == [5, 6, 7] and len(loader) == 3 and len(batches) == 3
    assert batches[0]["loss_mask"].sum() == 9 and (batches[0]["document_ids"][0, 9:] == -1).all()
