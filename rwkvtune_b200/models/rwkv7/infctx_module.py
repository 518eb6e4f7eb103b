"""State containers for infinite-context (chunked) training.

Same shapes and accessors as ``rwkvtune/models/rwkv7/infctx_module.py:49-201``:
``shift_states [L, 2, B, C]`` in the model dtype (index 0 = time-mix, 1 = channel-mix
carried row) and ``wkv_states [L, B, H, N, N]`` in fp32.
"""
from __future__ import annotations

import torch


class TimeMixState:
    def __init__(self, shift_state: torch.Tensor, wkv_state: torch.Tensor):
        self.shift_state = shift_state
        self.wkv_state = wkv_state


class ChannelMixState:
    def __init__(self, shift_state: torch.Tensor):
        self.shift_state = shift_state


class BlockState:
    def __init__(self, time_mix_state: TimeMixState, channel_mix_state: ChannelMixState):
        self.time_mix_state = time_mix_state
        self.channel_mix_state = channel_mix_state


class BlockStateList:
    def __init__(self, shift_states: torch.Tensor, wkv_states: torch.Tensor):
        self.shift_states = shift_states
        self.wkv_states = wkv_states

    @staticmethod
    def create(n_layer: int, batch_size: int, n_embd: int, n_head: int, device, dtype=torch.bfloat16,
               head_size: int = None):
        batch = batch_size
        N = head_size if head_size is not None else n_embd // n_head
        return BlockStateList(
            torch.zeros(n_layer, 2, batch, n_embd, device=device, dtype=dtype),
            torch.zeros(n_layer, batch, n_head, N, N, device=device, dtype=torch.float32),
        )

    @staticmethod
    def empty(n_layer: int, batch_size: int, n_embd: int, n_head: int, device, dtype=torch.bfloat16,
              head_size: int = None):
        batch = batch_size
        N = head_size if head_size is not None else n_embd // n_head
        return BlockStateList(
            torch.empty(n_layer, 2, batch, n_embd, device=device, dtype=dtype),
            torch.empty(n_layer, batch, n_head, N, N, device=device, dtype=torch.float32),
        )

    def __len__(self) -> int:
        return self.shift_states.shape[0]

    def __getitem__(self, layer: int) -> BlockState:
        return BlockState(TimeMixState(self.shift_states[layer, 0], self.wkv_states[layer]),
                          ChannelMixState(self.shift_states[layer, 1]))

    def __setitem__(self, layer: int, state: BlockState) -> None:
        self.shift_states[layer, 0] = state.time_mix_state.shift_state
        self.wkv_states[layer] = state.time_mix_state.wkv_state
        self.shift_states[layer, 1] = state.channel_mix_state.shift_state

    def detach(self) -> "BlockStateList":
        return BlockStateList(self.shift_states.detach(), self.wkv_states.detach())

    def to(self, device) -> "BlockStateList":
        return BlockStateList(self.shift_states.to(device), self.wkv_states.to(device))

    def clone(self) -> "BlockStateList":
        return BlockStateList(self.shift_states.clone(), self.wkv_states.clone())
