"""Command-line flags flow into the trainers' loss settings, and the per-algorithm defaults
of the decoder-shaping flags (parity with the reference CLI)."""

import argparse

import pytest

from speculators_b200 import losses
from speculators_b200.losses import eager
from speculators_b200.models.dflash.core import DFlashDraftModel
from speculators_b200.models.dspark.core import DSparkDraftModel
from speculators_b200.models.eagle3.core import Eagle3DraftModel
from speculators_b200.models.peagle.core import PEagleDraftModel
from speculators_b200.train.config import TrainConfig


def _parse(extra):
    cfg = TrainConfig.resolve(["--verifier-name-or-path", "dummy", *extra])
    return argparse.Namespace(**cfg.flatten())


def test_dflash_loss_flags():
    train_kw, val_kw = DFlashDraftModel.get_trainer_kwargs(**vars(_parse([])))
    assert train_kw["loss_config"]["kl_div"][0] is losses.kl_div_loss and "kl_div" in val_kw["loss_config"]
    assert train_kw["gamma"] == 4.0 and val_kw["gamma"] == 4.0
    train_kw, val_kw = DFlashDraftModel.get_trainer_kwargs(**vars(_parse(["--loss-fn", "ce"])))
    assert train_kw["loss_config"]["ce"][0] is losses.ce_loss and "ce" in val_kw["loss_config"]
    train_kw, val_kw = DFlashDraftModel.get_trainer_kwargs(**vars(_parse(["--dflash-decay-gamma", "7.0"])))
    assert train_kw["gamma"] == 7.0 and val_kw["gamma"] == 7.0
    train_kw, _ = DFlashDraftModel.get_trainer_kwargs(loss_fn="kl_div")
    assert train_kw["gamma"] == 4.0
    train_kw, val_kw = DFlashDraftModel.get_trainer_kwargs(**vars(_parse(["--loss-fn", '{"ce": 0.1, "tv": 0.9}'])))
    assert train_kw["loss_config"]["ce"][1] == 0.1 and train_kw["loss_config"]["tv"][1] == 0.9
    assert {"ce", "tv"} <= set(val_kw["loss_config"])


@pytest.mark.parametrize("model", [Eagle3DraftModel, PEagleDraftModel])
def test_eagle_family_loss_flags(model):
    train_kw, val_kw = model.get_trainer_kwargs(**vars(_parse([])))
    assert train_kw["loss_config"]["kl_div"][0] is losses.kl_div_loss and "kl_div" in val_kw["loss_config"]
    train_kw, _ = model.get_trainer_kwargs(**vars(_parse(["--loss-fn", "ce"])))
    assert train_kw["loss_config"]["ce"][0] is losses.ce_loss


def test_dspark_loss_flags():
    train_kw, val_kw = DSparkDraftModel.get_trainer_kwargs(**vars(_parse([])))
    assert train_kw["loss_config"]["kl_div"][0] is losses.kl_div_loss and train_kw["tv_loss_fn"] is losses.tv_loss
    assert train_kw["confidence_head_alpha"] == 1.0 and val_kw["confidence_head_alpha"] == 1.0
    train_kw, val_kw = DSparkDraftModel.get_trainer_kwargs(**vars(_parse(["--loss-implementation", "eager"])))
    assert train_kw["loss_config"]["kl_div"][0] is eager.kl_div_loss
    assert train_kw["tv_loss_fn"] is eager.tv_loss and val_kw["tv_loss_fn"] is eager.tv_loss
    train_kw, _ = DSparkDraftModel.get_trainer_kwargs(**vars(_parse(["--loss-fn", '{"ce": 0.1, "tv": 0.9}'])))
    assert train_kw["loss_config"]["ce"] == (losses.ce_loss, 0.1) or list(train_kw["loss_config"]["ce"]) == [losses.ce_loss, 0.1]
    assert train_kw["loss_config"]["tv"][0] is losses.tv_loss and train_kw["loss_config"]["tv"][1] == 0.9
    train_kw, val_kw = DSparkDraftModel.get_trainer_kwargs(**vars(_parse(["--confidence-head-alpha", "0.5"])))
    assert train_kw["confidence_head_alpha"] == 0.5 and val_kw["confidence_head_alpha"] == 0.5


def test_per_algorithm_defaults():
    e = _parse([])
    assert (e.draft_arch, e.norm_before_fc, e.norm_output) == ("llama", True, True)
    assert (e.num_layers, e.per_position_loss_weight, e.loss_fn, e.block_size) == (1, "fixed-exp-decay", "kl_div", 8)
    d = _parse(["--speculator-type", "dflash"])
    assert (d.draft_arch, d.norm_before_fc, d.norm_output) == ("qwen3", False, False)
    assert (d.num_layers, d.per_position_loss_weight, d.loss_fn, d.block_size) == (5, "dpace", "ce", 16)
    assert _parse(["--speculator-type", "dspark"]).block_size == 8
    o = _parse(["--speculator-type", "dflash", "--num-layers", "3", "--per-position-loss-weight", "fixed-exp-decay", "--loss-fn", "kl_div",
                "--block-size", "8"])
    assert (o.num_layers, o.per_position_loss_weight, o.loss_fn, o.block_size) == (3, "fixed-exp-decay", "kl_div", 8)
    assert _parse(["--no-norm-before-fc"]).norm_before_fc is False
    assert _parse(["--no-norm-output"]).norm_output is False


def test_max_steps_flag():
    assert _parse([]).max_steps is None
    assert _parse(["--max-steps", "15"]).max_steps == 15
    with pytest.raises(SystemExit):
        _parse(["--max-steps", "0"])
