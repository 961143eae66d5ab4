"""Multipack data-loader plugin - needs BOTH ``training.dataloader.multipack`` and ``training.attention``.

Behaviour of fms_acceleration_aadp/framework_plugin_multipack.py:31-183 in the reference: only for
distributed, padding-free training; the training ``DataLoader`` is replaced (and the accelerator's own
``prepare`` skipped) by one driven by ``MultipackDistributedBatchSampler`` with capacity
``per_device_train_batch_size * mean(token length)``, seed 42; token lengths are computed on rank 0 first.
"""
from __future__ import annotations

import warnings
from types import MethodType
from typing import Dict, Tuple

import torch
from torch.utils.data import DataLoader

from ...framework.framework_plugin import AccelerationPlugin


class MultipackDataloaderAccelerationPlugin(AccelerationPlugin):
    # the allocator is compiled in-tree (C++); numba is not needed
    require_packages = None

    def __init__(self, configurations: Dict[str, Dict], seed: int = 42):
        super().__init__(configurations)
        self.num_processes = self._check_config_and_maybe_check_values(key="training.dataloader.multipack.num_processes")
        attention = self._check_config_and_maybe_check_values(key="training.attention")
        self._seed = seed
        self._padding_free = False
        self._pad_token_id = None
        if "padding_free" in attention:
            self._padding_free = True
        else:
            assert self._pad_token_id is not None, "need to get pad token id"

    @property
    def requires_augmentation(self):
        return True

    def augmentation(self, model, train_args, modifiable_args: Tuple):
        from ...framework.accelerator_patcher import AcceleratorPatcher, AcceleratorPatcherComponent
        from .aadp_utils import calculate_token_lengths
        from .multipack_sampler import MultipackDistributedBatchSampler

        if not (torch.distributed.is_available() and torch.distributed.is_initialized()):
            raise AssertionError("Multipack dataloader only works for distributed training.")
        num_bins = torch.distributed.get_world_size()
        rank = torch.distributed.get_rank()

        def _prereq(dataloader: DataLoader) -> bool:
            return hasattr(dataloader, "dataset")

        def _build_multipack_dataloader(dataloader: DataLoader, accelerator):
            assert not getattr(accelerator.state, "deepspeed_plugin", None), \
                "Currently, multipack not supported for deepspeed"
            dataset = dataloader.dataset
            # rank 0 maps the dataset first so the others can reuse its cache
            if rank > 0:
                warnings.warn("Waiting for main process to perform the mapping. If the dataset is large, some "
                              "processes might time out; increase the timeout or the number of workers "
                              f"(> {self.num_processes}).")
                torch.distributed.barrier()
            lengths = calculate_token_lengths(dataset, num_processes=self.num_processes)
            if rank == 0:
                torch.distributed.barrier()
            self._max_number_tokens = train_args.per_device_train_batch_size * lengths.mean()
            sampler = MultipackDistributedBatchSampler(
                batch_max_length=self._max_number_tokens, lengths=lengths, num_replicas=num_bins, rank=rank,
                seed=self._seed, padding=not self._padding_free)
            new_loader = DataLoader(dataset, batch_sampler=sampler, num_workers=dataloader.num_workers,
                                    collate_fn=dataloader.collate_fn)

            def _set_epoch(self, epoch: int):
                self.batch_sampler.set_epoch(epoch)

            new_loader.set_epoch = MethodType(_set_epoch, new_loader)
            return new_loader

        AcceleratorPatcher.replace("multipack", AcceleratorPatcherComponent.data_loader,
                                   replacement_builder=_build_multipack_dataloader, pre_requisite_check=_prereq,
                                   skip_prepare=True)
        self._train_args = train_args
        return model, modifiable_args


AccelerationPlugin.register_plugin(
    MultipackDataloaderAccelerationPlugin,
    configuration_and_paths=["training.dataloader.multipack", "training.attention"],
)
