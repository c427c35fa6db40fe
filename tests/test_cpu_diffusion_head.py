"""Host arithmetic of the diffusion head and the sampler loop (reference: nn/d_diffusion_head.py:172-227,
d_alphafold3.py:316-404) against the oracle's line-by-line restatement, on CPU tensors (element-wise plumbing,
no kernel is involved).  The denoiser is a stand-in: the token-level transformer is covered by the GPU tests."""
import pytest
import torch


@pytest.fixture(scope="module")
def dh(pkg):
    from distributed_xfold_b200 import diffusion_head
    return diffusion_head


def schedule_standin(t):
    """Any decreasing positive schedule will do here: the reference takes its own from the absent xfold package."""
    return 160.0 * (0.0004 / 160.0) ** t


def test_edm_mix_and_scalings(dh, oracle):
    g = torch.Generator().manual_seed(1)
    noisy = torch.randn(3, 20, 24, 3, generator=g, dtype=torch.float64)
    upd = torch.randn(3, 20, 24, 3, generator=g, dtype=torch.float64)
    mask = (torch.rand(20, 24, generator=g) > 0.3).double()[None]
    for t in (0.0004, 1.0, 16.0, 160.0):
        t = torch.tensor(t, dtype=torch.float64)
        got = dh.denoised_positions(noisy, upd, t, mask)
        ref = oracle.diffusion_head_mix(noisy, upd, t, mask)
        assert torch.allclose(got, ref, rtol=1e-12, atol=1e-12)
        assert torch.allclose(dh.input_scaling(t), 1 / torch.sqrt(t ** 2 + 16.0 ** 2))
        assert torch.allclose(dh.fourier_argument(t), 0.25 * torch.log(t / 16.0))
    # at sigma = SIGMA_DATA the two branches weigh 1/2 and sigma / sqrt(2)
    t = torch.tensor(16.0, dtype=torch.float64)
    one = torch.ones(1, 1, 1, 3, dtype=torch.float64)
    assert torch.allclose(dh.denoised_positions(one, one, t, torch.ones(1, 1, 1, dtype=torch.float64)),
                          (0.5 + 16.0 / 2 ** 0.5) * one)


def test_sampler_constants(dh, oracle):
    levels = schedule_standin(torch.linspace(0, 1, 201, dtype=torch.float64))
    s = dh.SamplerSchedule(levels)
    nl, th, ns = oracle.sampler_constants(levels)
    assert s.steps == 200
    assert torch.equal(s.noise_level, nl) and torch.equal(s.t_hat, th) and torch.equal(s.noise_scale, ns)
    # gamma switches off once the level falls to gamma_min: t_hat equals the previous level there and no noise is added
    low = levels[1:] <= 1.0
    assert torch.equal(s.t_hat[low], levels[:-1][low]) and float(s.noise_scale[low].abs().max()) == 0.0
    assert torch.allclose(s.t_hat[~low], 1.8 * levels[:-1][~low])


@pytest.mark.parametrize("num_samples,dp,expect", [(1, 1, False), (5, 1, True), (5, 5, False), (8, 4, True), (8, 8, False)])
def test_batch_infer_rule(dh, num_samples, dp, expect):
    assert dh.use_batch_infer(num_samples, dp) is expect


def test_sample_split_follows_shardinfo(dh):
    # the reference's rule as it stands (distribute_utils.py:107-121): ceil(5 / 4) = 2 for the first three ranks and
    # 5 % 2 = 1 for the last, which over-covers 5 samples; sizes that divide, or leave at most one short shard, are exact
    assert [dh.local_sample_count(5, 4, r, True) for r in range(4)] == [2, 2, 2, 1]
    assert [dh.local_sample_count(5, 2, r, True) for r in range(2)] == [3, 2]
    assert [dh.local_sample_count(8, 4, r, True) for r in range(4)] == [2, 2, 2, 2]
    assert dh.local_sample_count(5, 4, 3, False) == 5


@pytest.mark.parametrize("num_samples,dp,rank", [(1, 1, 0), (5, 1, 0), (5, 2, 1)])
def test_sampler_loop_matches_oracle(dh, oracle, num_samples, dp, rank):
    levels = schedule_standin(torch.linspace(0, 1, 21, dtype=torch.float64))
    mask = torch.ones(7, 5, dtype=torch.float64)
    target = torch.randn(7, 5, 3, generator=torch.Generator().manual_seed(3), dtype=torch.float64)

    def denoiser(noisy, t_hat, step):  # a contraction towards a fixed structure, EDM-mixed like the head's output
        return dh.denoised_positions(noisy, (target - noisy) / 4.0, t_hat, mask)

    got = dh.sample_diffusion(denoiser, dh.SamplerSchedule(levels), mask, num_samples, dp_size=dp, dp_rank=rank,
                              use_dp=dp > 1, generator=torch.Generator().manual_seed(9))
    batch = dh.use_batch_infer(num_samples, dp)
    n_local = dh.local_sample_count(num_samples, dp, rank, dp > 1) if batch else 1
    assert got.shape == (n_local, 7, 5, 3)
    shape = ((n_local,) if batch else ()) + (7, 5, 3)
    p0 = torch.randn(shape, generator=torch.Generator().manual_seed(9)) * levels[0]
    ref = oracle.sample_diffusion(denoiser, levels, p0)
    ref = ref if batch else ref[None]
    assert torch.allclose(got, ref, rtol=1e-10, atol=1e-10)
    assert torch.isfinite(got).all()
