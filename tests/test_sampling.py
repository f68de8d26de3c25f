"""The host sampler against the reference's rules (src/model.cpp:667-757)."""
import numpy as np

from exl3_server_b200.sampling import SampleOptions, SplitMix64, apply_penalties, sample_token


def test_splitmix64_known_values():
    # first outputs of splitmix64 from state 0 (public test vector of the generator)
    g = SplitMix64(0)
    assert [g.next() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    u = SplitMix64(123).uniform01()
    assert 0.0 <= u < 1.0


def test_greedy_takes_the_first_maximum():
    logits = np.array([0.5, 2.0, 2.0, -1.0], dtype=np.float32)
    assert sample_token(logits, SampleOptions(), [], SplitMix64(1)) == 1


def test_penalties():
    logits = np.array([2.0, -2.0, 1.0, 1.0], dtype=np.float32)
    opt = SampleOptions(repetition_penalty=2.0, presence_penalty=0.5, frequency_penalty=0.25)
    apply_penalties(logits, opt, [0, 1, 1, 9, -3])
    # token 0 seen once: 2/2 - 0.5 - 0.25; token 1 seen twice: -2*2 - 0.5 - 0.5
    assert np.allclose(logits, [0.25, -5.0, 1.0, 1.0])


def test_top_k_top_p_min_p_limit_the_support():
    logits = np.log(np.array([0.5, 0.25, 0.15, 0.07, 0.03], dtype=np.float32))

    def support(opt):
        g = SplitMix64(7)
        return {sample_token(logits, opt, [], g) for _ in range(600)}

    assert support(SampleOptions(temperature=1.0)) == {0, 1, 2, 3, 4}
    assert support(SampleOptions(temperature=1.0, top_k=2)) == {0, 1}
    assert support(SampleOptions(temperature=1.0, top_p=0.7)) == {0, 1}          # 0.5 + 0.25 >= 0.7
    assert support(SampleOptions(temperature=1.0, min_p=0.4)) == {0, 1}          # p >= 0.4 * 0.5
    assert support(SampleOptions(temperature=1.0, min_p=0.4, top_k=1)) == {0}


def test_distribution_follows_temperature():
    logits = np.log(np.array([0.6, 0.3, 0.1], dtype=np.float32))
    g = SplitMix64(99)
    n = 20000
    counts = np.bincount([sample_token(logits, SampleOptions(temperature=1.0), [], g) for _ in range(n)], minlength=3)
    assert np.allclose(counts / n, [0.6, 0.3, 0.1], atol=0.015)
    g = SplitMix64(99)
    counts = np.bincount([sample_token(logits, SampleOptions(temperature=0.5), [], g) for _ in range(n)], minlength=3)
    p = np.array([0.36, 0.09, 0.01]) / 0.46
    assert np.allclose(counts / n, p, atol=0.015)


def test_candidate_cap_of_2048():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=5000).astype(np.float32)
    order = np.argsort(-logits)
    allowed = set(order[:2048].tolist())
    g = SplitMix64(3)
    picks = {sample_token(logits, SampleOptions(temperature=50.0), [], g) for _ in range(3000)}
    assert picks <= allowed and len(picks) > 1000


def test_equal_logits_rank_by_index():
    # 3000 tokens share the largest value: the candidates are the 2048 with the smallest indices, in index order
    logits = np.zeros(5000, dtype=np.float32)
    logits[1000:4000] = 1.0

    class U:
        def __init__(self, u):
            self.u = u

        def uniform01(self):
            return self.u

    opt = SampleOptions(temperature=1.0)
    assert sample_token(logits, opt, [], U(0.0)) == 1000
    assert sample_token(logits, opt, [], U(0.999999)) == 1000 + 2047
    assert sample_token(logits, opt, [], U(0.5)) in (1000 + 1023, 1000 + 1024)
    assert sample_token(logits, SampleOptions(temperature=1.0, top_k=3), [], U(0.99)) == 1002
