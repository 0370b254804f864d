"""Mooncake backend: hidden states travel through a Mooncake distributed store, so
producer and trainer need no shared filesystem (flags and ``kv_transfer_config``
shape: hs_connectors/src/hs_connectors/transfer.py:211-334)."""

from __future__ import annotations

import argparse
import dataclasses
import os
import socket
from typing import Any

import torch

from speculators_b200.hs_connectors.store import HiddenStatesStore, MooncakeStoreConfig
from speculators_b200.hs_connectors.transfer import HiddenStatesBackend, HiddenStatesTransfer

__all__ = ["MooncakeBackend", "MooncakeTransfer"]


def _local_hostname() -> str:
    explicit = os.environ.get("MOONCAKE_LOCAL_HOSTNAME")
    if explicit:
        return explicit
    try:
        return socket.gethostbyname(socket.gethostname())
    except OSError:
        return "127.0.0.1"


class MooncakeTransfer(HiddenStatesTransfer):
    def __init__(self, store: HiddenStatesStore):
        self.store = store

    def setup(self) -> None:
        if not self.store.is_setup:
            self.store.setup()

    def get_cached(self, file_idx: int) -> dict[str, torch.Tensor] | None:  # noqa: ARG002
        return None

    def get_generated(self, handle: str) -> dict[str, torch.Tensor] | None:
        return self.store.get_sample(handle)

    def delete(self, handle: str) -> None:
        self.store.delete_sample(handle)


def _config_from(args: argparse.Namespace, **extra: Any) -> MooncakeStoreConfig:
    return MooncakeStoreConfig(
        local_hostname=_local_hostname(), metadata_server=args.mooncake_metadata_server,
        master_server_address=args.mooncake_master,
        global_segment_size=round(args.mooncake_global_segment_gib * 1024**3),
        local_buffer_size=round(args.mooncake_local_buffer_gib * 1024**3), protocol=args.mooncake_protocol, **extra,
    )


@HiddenStatesBackend.register("mooncake")
class MooncakeBackend(HiddenStatesBackend):
    @staticmethod
    def _common(parser: argparse.ArgumentParser) -> None:
        parser.add_argument("--mooncake-master", type=str, default="127.0.0.1:50051", help="Mooncake master server address.")
        parser.add_argument("--mooncake-metadata-server", type=str, default="P2PHANDSHAKE", help="Mooncake metadata server (or P2PHANDSHAKE).")
        parser.add_argument("--mooncake-protocol", choices=["tcp", "rdma"], default="tcp", help="Mooncake transport protocol.")
        parser.add_argument("--mooncake-global-segment-gib", type=float, default=4.0, help="Memory each client registers for globally visible objects, GiB.")
        parser.add_argument("--mooncake-local-buffer-gib", type=float, default=2.0, help="Client-local staging buffer, GiB.")

    @staticmethod
    def add_train_args(parser: argparse.ArgumentParser) -> None:
        MooncakeBackend._common(parser)

    @staticmethod
    def add_launch_args(parser: argparse.ArgumentParser) -> None:
        MooncakeBackend._common(parser)
        parser.add_argument("--mooncake-writer-threads", type=int, default=4, help="Asynchronous writer threads in the producer.")

    @staticmethod
    def from_train_args(args: argparse.Namespace, data_path: str) -> MooncakeTransfer:  # noqa: ARG004
        return MooncakeTransfer(HiddenStatesStore(_config_from(args)))

    @staticmethod
    def build_kv_transfer_config(args: argparse.Namespace) -> dict[str, Any]:
        cfg = _config_from(args, num_writer_threads=args.mooncake_writer_threads)
        return {
            "kv_connector": "MooncakeHiddenStatesConnector",
            "kv_role": "kv_producer",
            "kv_connector_module_path": "speculators_b200.hs_connectors.vllm_connector",
            "kv_connector_extra_config": {"mooncake": dataclasses.asdict(cfg)},
        }
