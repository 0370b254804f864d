"""The documentation names real things: every train.py flag is documented and every
documented flag exists; the YAML example resolves; relative links point at files."""

import re
from pathlib import Path

import pytest

DOCS = Path(__file__).resolve().parent.parent / "docs"


def _parser_flags() -> set[str]:
    from speculators_b200.train.config.resolution import build_parser

    flags: set[str] = set()
    for action in build_parser()._actions:  # noqa: SLF001
        flags.update(o for o in action.option_strings if o.startswith("--") and o != "--help")
    return flags


def test_train_flag_reference_matches_the_parser():
    text = (DOCS / "cli" / "train.md").read_text()
    table = text[text.index("## Flags"):text.index("## What a run writes")]
    documented = set(re.findall(r"`(--[a-z0-9-]+)`", table))
    flags = _parser_flags()
    assert flags - documented == set(), f"flags missing from docs/cli/train.md: {sorted(flags - documented)}"
    assert documented - flags == set(), f"docs/cli/train.md names flags the parser does not have: {sorted(documented - flags)}"


def test_yaml_example_resolves(tmp_path):
    from speculators_b200.train.config.resolution import resolve
    from speculators_b200.train.config.schema import TrainConfig

    text = (DOCS / "cli" / "train.md").read_text()
    example = re.search(r"```yaml\n(.*?)```", text, re.S).group(1)
    path = tmp_path / "run.yaml"
    path.write_text(example)
    cfg = resolve(TrainConfig, ["--config", str(path)])
    assert cfg.speculator_type == "dflash"
    assert cfg.dflash.block_size == 16 and cfg.dflash.per_position_loss_weight == "dpace"
    assert cfg.draft.target_layer_ids == [2, 18, 33] and cfg.trainer.fsdp_shard is True


def test_flags_used_in_tutorials_exist():
    flags = _parser_flags()
    text = (DOCS / "user_guide" / "tutorials" / "train.md").read_text()
    blocks = re.findall(r"```bash\n(.*?)```", text, re.S)
    used: set[str] = set()
    for block in blocks:
        # only the train.py invocations: commands of other scripts carry their own flags
        for chunk in re.split(r"\n(?=\S)", block):
            if "train.py" in chunk or chunk.lstrip().startswith("..."):
                used.update(re.findall(r"(--[a-z][a-z0-9_-]+)", chunk))
    launcher = {"--standalone", "--nproc_per_node", "--nproc-per-node"}
    unknown = {f for f in used if f not in flags and f not in launcher}
    assert not unknown, f"the training tutorial uses flags train.py does not have: {sorted(unknown)}"


@pytest.mark.parametrize("page", sorted(str(p.relative_to(DOCS)) for p in DOCS.rglob("*.md")))
def test_relative_links_resolve(page):
    path = DOCS / page
    for target in re.findall(r"\]\(([^)#]+)(?:#[^)]*)?\)", path.read_text()):
        if "://" in target:
            continue
        assert (path.parent / target).exists(), f"{page}: broken link {target}"
