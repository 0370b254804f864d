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


def test_packed_ring_sample_equals_collated_documents():
    """Several documents run through the verifier as one packed row: the device-side builder must give the
    batch the file path collates from the documents' separate samples (incl. clipping at the packed length)."""
    H, layers = 8, 4
    for lens, seq_len in (((7, 12, 9), 32), ((7, 12, 9), 20), ((5,), 8), ((3, 1, 6), 16)):
        docs = [_sample(n, layers, H, seed=10 * n + i) for i, n in enumerate(lens)]
        items = []
        for stored, ids, mask in docs:
            aux, last = split_hidden_state_layers(stored)
            items.append({"hidden_states": aux, "input_ids": ids, "verifier_last_hidden_states": last, "loss_mask": mask,
                          "lengths": torch.tensor([ids.shape[0]]), "position_ids": torch.arange(ids.shape[0])})
        want = CollateFn(seq_len, H, layers - 1, torch.bfloat16, preprocess=shift_batch)(items)
        packed = {"hidden_states": torch.cat([d[0] for d in docs]).flatten(1), "token_ids": torch.cat([d[1] for d in docs])}
        got = batch_from_ring_sample(packed, H, seq_len, loss_mask=torch.cat([d[2] for d in docs]), lengths=list(lens))
        for key in want:
            assert torch.equal(got[key].to(want[key].dtype), want[key]), (lens, seq_len, key)


def test_ring_batch_loader_takes_mask_and_lengths_from_the_plan():
    class FakeRing:
        def pop(self, seq, timeout_s):
            stored, ids, _ = _sample(12, seed=seq)
            return {"hidden_states": stored.flatten(1), "token_ids": ids}

    seen = []

    def meta(i):
        seen.append(i)
        return torch.ones(12, dtype=torch.bool), [5, 7]

    loader = RingBatchLoader(FakeRing(), num_steps=2, hidden_size=8, seq_len=16, meta_fn=meta)
    first, second = list(loader)
    assert seen == [0, 1]
    assert first["document_ids"][0].tolist() == [0] * 4 + [1] * 6 + [-1] * 6
    assert first["position_ids"][0, :10].tolist() == [1, 2, 3, 4, 1, 2, 3, 4, 5, 6] and int(second["loss_mask"].sum()) == 10
