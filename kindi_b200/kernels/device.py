"""What the choice of kernels assumes about the GPU: one place for the numbers of the cost estimates.

The estimates only rank alternatives that are all correct (tile widths, ways to split K, one CTA or a pair per tile),
so a number that is off costs speed, never a result. What the device reports about itself is read from it (number
of SMs, size of the L2); the rates are measurements on a B200 and are named for what they measure, so that another
GPU's figures can be put in their place.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class DeviceModel:
    n_sm: int = 148                      # B200: 2 dies x 74 SMs
    l2_bytes: int = 126 * 2 ** 20        # both halves of the L2
    hbm_bytes_per_us: float = 6.6e6      # a streaming kernel's rate over all SMs (copy bandwidth, 6.6 TB/s)
    # one K block (64 deep) of a 128 x 256 tile on one SM's tensor cores, in microseconds (1.5 PFLOP/s over 148 SMs)
    mma_us_per_kblock_128x256: float = 0.276
    # bringing one 128-byte operand row of a K block from the L2 into an SM's shared memory, in microseconds
    l2_us_per_operand_row: float = 1.15e-3
    # a K block of a 256 x 256 tile on a pair of SMs (cta_group::2), measured 0.36-0.39; narrower tiles not below 0.33
    pair_us_per_kblock_256x256: float = 0.37
    pair_us_per_kblock_floor: float = 0.33
    # operands of a product whose K blocks are dealt out over all pairs have to stay in the L2 meanwhile; beyond this
    # many bytes the product waits for DRAM (measured: 5120 x 13824 weights, 288 us against 226)
    l2_resident_bytes: float = 100e6

    @staticmethod
    def current() -> "DeviceModel":
        try:
            if torch.cuda.is_available():
                p = torch.cuda.get_device_properties(torch.cuda.current_device())
                return DeviceModel(n_sm=p.multi_processor_count,
                                   l2_bytes=int(getattr(p, "L2_cache_size", 0)) or DeviceModel.l2_bytes,
                                   l2_resident_bytes=0.8 * (int(getattr(p, "L2_cache_size", 0)) or DeviceModel.l2_bytes))
        except Exception:                                       # noqa: BLE001
            pass
        return DeviceModel()


DEVICE = DeviceModel.current()
