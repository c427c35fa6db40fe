"""Host-side arithmetic of the diffusion head around the DiffusionTransformer
(reference: nn/d_diffusion_head.py:172-227 and the sampler d_alphafold3.py:316-404).

What is here is what the reference states itself:

* the EDM pre-conditioning of the denoiser (SIGMA_DATA = 16, nn/d_diffusion_head.py:44): input scaling
  ``1 / sqrt(t^2 + sigma^2)``, and the skip / output mix of the prediction (:216-227);
* the sampler's step arithmetic: ``gamma``, ``t_hat``, ``noise_scale`` per step from a noise schedule
  (d_alphafold3.py:366-375), the Euler step with ``step_scale`` (:343-347), the initial draw (:384-397);
* the ``batch_infer`` rule (:273) and the split of the samples over the ranks by ShardInfo (:381-385);
* the Fourier feature argument ``log(t / sigma) / 4`` of the noise embedding (nn/d_diffusion_head.py:128-130).

What the reference takes from the absent ``xfold`` package is passed in: the noise schedule
(``diffusion_head.noise_schedule``), the random augmentation of the positions, and the denoiser's atom
encoder / decoder.  The denoiser argument is any callable ``(positions_noisy, t_hat, step_index) -> positions``;
the token-level part of it is ``diffusion.PackedDiffusionTransformer`` on the sm_100a kernels.

Positions are a few MB: this is element-wise plumbing on whatever device the tensors live on, not a kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .distribute_utils import ShardInfo

SIGMA_DATA = 16.0  # nn/d_diffusion_head.py:44


def input_scaling(noise_level: torch.Tensor) -> torch.Tensor:
    """Factor applied to the masked noisy positions before the atom encoder (nn/d_diffusion_head.py:186-187)."""
    return torch.rsqrt(noise_level ** 2 + SIGMA_DATA ** 2)


def fourier_argument(noise_level: torch.Tensor) -> torch.Tensor:
    """Argument of the noise-level Fourier embedding (nn/d_diffusion_head.py:128-130)."""
    return 0.25 * torch.log(noise_level / SIGMA_DATA)


def denoised_positions(positions_noisy: torch.Tensor, position_update: torch.Tensor, noise_level: torch.Tensor,
                       atom_mask: torch.Tensor) -> torch.Tensor:
    """skip_scaling * positions_noisy + out_scaling * position_update, masked (nn/d_diffusion_head.py:216-227).
    atom_mask broadcasts against the positions without their last axis."""
    skip = SIGMA_DATA ** 2 / (noise_level ** 2 + SIGMA_DATA ** 2)
    out = noise_level * SIGMA_DATA * torch.rsqrt(noise_level ** 2 + SIGMA_DATA ** 2)
    return (skip * positions_noisy + out * position_update) * atom_mask[..., None]


@dataclass
class SamplerSchedule:
    """Per-step constants of the sampler (d_alphafold3.py:262-265, 363-375)."""
    noise_levels: torch.Tensor  # [steps + 1], from the noise schedule
    gamma_0: float = 0.8
    gamma_min: float = 1.0
    noise_scale_factor: float = 1.003
    step_scale: float = 1.5

    def __post_init__(self):
        prev, cur = self.noise_levels[:-1], self.noise_levels[1:]
        gamma = self.gamma_0 * (cur > self.gamma_min)
        self.noise_level = cur
        self.t_hat = prev * (1 + gamma)
        self.noise_scale = self.noise_scale_factor * torch.sqrt(self.t_hat ** 2 - prev ** 2)

    @property
    def steps(self) -> int:
        return self.noise_level.shape[0]


def use_batch_infer(num_samples: int, dp_size: int) -> bool:
    """Several samples per rank go through the denoiser as one batch (d_alphafold3.py:273)."""
    return num_samples != 1 and num_samples != dp_size


def local_sample_count(num_samples: int, dp_size: int, dp_rank: int, use_dp: bool) -> int:
    """Samples this rank draws (d_alphafold3.py:381-388)."""
    if not use_dp:
        return num_samples
    return ShardInfo(num_samples, dp_size).get_shard_size_list()[dp_rank]


def euler_step(positions_noisy: torch.Tensor, positions_denoised: torch.Tensor, noise_level: torch.Tensor,
               t_hat: torch.Tensor, step_scale: float) -> torch.Tensor:
    """d_alphafold3.py:343-347."""
    grad = (positions_noisy - positions_denoised) / t_hat
    return positions_noisy + step_scale * (noise_level - t_hat) * grad


def sample_diffusion(denoiser: Callable[[torch.Tensor, torch.Tensor, int], torch.Tensor], schedule: SamplerSchedule,
                     atom_mask: torch.Tensor, num_samples: int, dp_size: int = 1, dp_rank: int = 0, use_dp: bool = False,
                     augment: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None,
                     generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """The loop of ``_sample_diffusion`` (d_alphafold3.py:316-404).  atom_mask: [num_token, num_atom].
    Returns [local samples, num_token, num_atom, 3].  As in the reference, the per-step perturbation is the
    scalar ``noise_scale`` itself (its ``randn`` draw is commented out there, :336-338)."""
    batch_infer = use_batch_infer(num_samples, dp_size)
    dev = atom_mask.device
    if not batch_infer:
        shape = tuple(atom_mask.shape) + (3,)
    else:
        shape = (local_sample_count(num_samples, dp_size, dp_rank, use_dp),) + tuple(atom_mask.shape) + (3,)
    positions = torch.randn(shape, device=dev, generator=generator) * schedule.noise_levels[0]
    mask = atom_mask[None] if batch_infer else atom_mask
    for i in range(schedule.steps):
        if augment is not None:
            positions = augment(positions, mask)
        noisy = positions + schedule.noise_scale[i]
        denoised = denoiser(noisy, schedule.t_hat[i], i)
        positions = euler_step(noisy, denoised, schedule.noise_level[i], schedule.t_hat[i], schedule.step_scale)
    return positions if batch_infer else positions[None]
