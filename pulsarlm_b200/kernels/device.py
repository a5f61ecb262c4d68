"""What the host-side cost estimates know of the device: one description object.

The attention part chooses how to split keys among CTAs by estimating times; every
figure those estimates use that belongs to the device rather than to the kernel's
shape lives here, with where it was measured, so that another device is another
instance and not an edit of the part.
"""

from __future__ import annotations

import dataclasses

import torch


@dataclasses.dataclass(frozen=True)
class DeviceDescription:
    """Figures of one GPU model as the engine's kernels see them."""

    name: str
    # What the split-key decode attention reaches when CTAs are many: a little under the
    # copy bandwidth (measured with that kernel at batch 64, 2,048 and 8,192 keys).
    stream_bytes_per_second: float
    # What one CTA of that kernel takes in when CTAs are few (two 8 KB tiles in flight per
    # warp against the memory's answer time).
    cta_bytes_per_second: float
    # With more than sixteen splits (no cluster: partial results through scratch) a CTA reaches this
    # fraction of that rate (fitted: batch 1 at 131,072 keys and head size 128 takes 90 us in 22
    # splits, 84 in 28, 87 in 37; at head size 64 57 us in 44 splits, 50 in 56).
    scratch_cta_fraction: float
    # Of the clusters of s > 4 CTAs that the occupancy query says fit at once, the fraction 1 - s x this
    # finds room inside a step, between the CTAs of the kernels before and after (fitted in the step,
    # 8B shape at 2,060 keys: batch 4 in 8 shares 1,750 us for 16 layers, in 6 1,657; batch 2 in 13
    # 1,696, in 11 1,607; batch 3 in 10 1,670, in 8 1,638; batch 16 in 2 1,946, unsplit 2,039).
    cluster_room_loss_per_cta: float
    round_seconds: float          # start and end of a round of CTAs of the decode kernel
    cluster_merge_seconds: float  # merging up to sixteen splits inside a thread-block cluster
    merge_kernel_seconds: float   # merging more splits through scratch and a second kernel,
    merge_split_seconds: float    # and what each split adds to that (the merge reads every split's partial row)
    # Prompt attention (tcgen05), head size 128: one key for one CTA, the fixed cost of a round
    # of CTAs, the merge launch, and the bandwidth its partial rows are written and read at.
    prefill_key_seconds: float
    prefill_round_seconds: float
    prefill_merge_seconds: float
    prefill_scratch_bytes_per_second: float


B200 = DeviceDescription(
    name="B200",
    stream_bytes_per_second=6.3e12,
    cta_bytes_per_second=36e9,
    scratch_cta_fraction=0.8,
    cluster_room_loss_per_cta=0.025,
    round_seconds=2e-6,
    cluster_merge_seconds=2e-6,
    merge_kernel_seconds=5e-6,
    merge_split_seconds=0.1e-6,
    prefill_key_seconds=17.3e-9,
    prefill_round_seconds=6e-6,
    prefill_merge_seconds=4e-6,
    prefill_scratch_bytes_per_second=4e12,
)

_DESCRIPTIONS: dict = {}


def describe(device: torch.device) -> DeviceDescription:
    """The description the estimates use for `device`: the engine runs on sm_100 only, so
    this is the B200's until another is registered with `register`."""
    return _DESCRIPTIONS.get(device, B200)


def register(device: torch.device, description: DeviceDescription) -> None:
    _DESCRIPTIONS[device] = description
