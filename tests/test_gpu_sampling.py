"""Embedding gather and greedy argmax (the first and last launches of a decode step) through the C ABI.
Cases follow the reference's suite (tests/test_kernels.cu:402-448 and :1724-1830): bit-exact gathers in
packed and strided rows, odd shapes; argmax on full-vocabulary random rows, crafted ties across every
reduction boundary, signed zeros, the NaN policy, vocabulary tails and tiny rows. Both are exact gates."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from redline_llm_b200 import kernels as K  # noqa: E402
from redline_llm_b200 import workloads as wl  # noqa: E402
from tests.gpu_util import dev, host  # noqa: E402

VOCAB = 151936


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def argmax(logits):
    rows, vocab = logits.shape
    out = torch.full((rows + 2,), -7, dtype=torch.int32, device="cuda")
    d = dev(logits)
    K.lib().rl_launch_greedy_argmax(out.data_ptr() + 4, d.data_ptr(), rows, vocab,
                                    torch.cuda.current_stream().cuda_stream)
    got = out.cpu().numpy()
    assert got[0] == -7 and got[-1] == -7
    return got[1:-1]


@pytest.mark.parametrize("rows", [1, 3, 64])
def test_argmax_random_full_vocab(own, rows):
    x = wl.normal_half(0xA46 + rows, rows * VOCAB).reshape(rows, VOCAB)
    assert np.array_equal(argmax(x), own.argmax(x))


def test_argmax_ties_resolve_to_lowest_index_across_every_boundary(own):
    rows = 12
    x = np.full((rows, VOCAB), 0xBC00, np.uint16)  # -1 everywhere
    one = 0x3C00
    pairs = [(5, 6), (7, 8), (255, 256), (2047, 2048), (18991, 18992), (18992 * 3 - 1, 18992 * 3),
             (100, VOCAB - 1), (0, VOCAB - 1), (VOCAB - 2, VOCAB - 1), (75968, 75969), (31, 32), (8 * 256 - 1, 8 * 256 * 3)]
    for r, (a, b) in enumerate(pairs):
        x[r, a] = one
        x[r, b] = one
    got = argmax(x)
    assert np.array_equal(got, [min(p) for p in pairs])
    assert np.array_equal(got, own.argmax(x))


def test_argmax_signed_zeros_and_nan_policy(own):
    x = np.full((6, 4096), 0xBC00, np.uint16)
    x[0, 10], x[0, 3] = 0x0000, 0x8000           # +0 and -0 compare equal: lowest index wins
    x[1, :] = 0x7E00                             # all NaN -> token 0
    x[2, :] = 0xFC00                             # all -inf -> token 0 through the tie-break
    x[3, :] = 0x7E00
    x[3, 77] = 0xFC00                            # NaN never wins: the single -inf does
    x[4, 5] = 0x7E00
    x[4, 900] = 0x4000                           # a NaN next to real values is ignored
    x[5, 4095] = 0x7C00                          # +inf in the last column
    got = argmax(x)
    assert np.array_equal(got, [3, 0, 0, 77, 900, 4095])
    assert np.array_equal(got, own.argmax(x))


@pytest.mark.parametrize("vocab", [1, 2, 7, 8, 9, 63, 64, 65, 1000, 2047, 2049, 151935])
def test_argmax_vocab_tails_and_tiny_rows(own, vocab):
    x = wl.uniform_half(0x7A1 + vocab, 3 * vocab, -4.0, 4.0).reshape(3, vocab)
    assert np.array_equal(argmax(x), own.argmax(x))


@pytest.mark.parametrize("stride", [1536, 2048])
def test_embed_gather_bit_exact_packed_and_strided(stride):
    rows, hidden, vocab = 65, 1536, 4000
    table = wl.uniform_half(0xE1, vocab * hidden, -1.0, 1.0).reshape(vocab, hidden)
    ids = wl.randint(0xE2, rows, 0, vocab - 1)
    ids[3] = 0                                   # a padded slot gathers row 0
    before = wl.uniform_half(0xE3, rows * stride, -1.0, 1.0).reshape(rows, stride)
    d_out = dev(before)
    K.launch_embed_gather(d_out, stride, dev(table), dev(ids), rows, hidden)
    after = host(d_out).reshape(rows, stride)
    assert np.array_equal(after[:, :hidden], table[ids])
    assert np.array_equal(after[:, hidden:], before[:, hidden:])


def test_embed_gather_odd_shapes_take_the_scalar_path():
    rows, hidden, vocab = 5, 37, 50
    table = wl.uniform_half(0xE4, vocab * hidden, -1.0, 1.0).reshape(vocab, hidden)
    ids = wl.randint(0xE5, rows, 0, vocab - 1)
    d_out = torch.full((rows * hidden + 4,), 0x1111, dtype=torch.int16, device="cuda")
    K.launch_embed_gather(d_out, hidden, dev(table), dev(ids), rows, hidden)
    got = host(d_out)
    assert np.array_equal(got[:rows * hidden].reshape(rows, hidden), table[ids])
    assert (got[rows * hidden:] == 0x1111).all()
