"""Checkpoint and resume through the C ABI (gl_save_state / gl_load_state): a network loaded from a
state file continues bit for bit like the one that wrote it -- weights, scalar biases, epoch counter
and, in reference mode, the pending deltas of a minibatch window left open at the end of an epoch."""
import numpy as np
import pytest

from conftest import bits, libc_srand

pytestmark = pytest.mark.gpu


def _data(rng, rows, n_in, n_out):
    x = rng.standard_normal((rows, n_in)).astype(np.float32)
    y = rng.uniform(0.05, 0.95, (rows, n_out)).astype(np.float32)
    return x, y


@pytest.mark.parametrize("mode_name", ["reference", "batched", "reference_dropout"])
def test_resume_equals_uninterrupted_run(g, tmp_path, mode_name):
    if g.device_count() < 1:
        pytest.fail("no sm_100 device visible")
    rng = np.random.default_rng(77)
    sizes = [6, 9, 5, 2]
    rows = 37  # not a multiple of the minibatch: reference mode carries an open window across epochs
    mode = g.MODE_BATCHED if mode_name == "batched" else g.MODE_REFERENCE
    # with dropout the state also holds every edge's own history length and last delta and the error
    # accumulators that survive a row; the node flags come from rand(), seeded per run below
    pdrop = [0.3, 0.3, 0.4] if mode_name == "reference_dropout" else 0.0
    d = g.make_desc(sizes, ["tanh", "sigmoid", "sigmoid"], "regression", batch=8, lr=0.05, momentum=0.7, mode=mode,
                    p_dropout=pdrop)
    x, y = _data(rng, rows, sizes[0], sizes[-1])
    w0 = rng.uniform(-0.4, 0.4, g.weight_count(d)).astype(np.float32)
    b0 = rng.uniform(-0.1, 0.1, len(sizes) - 2).astype(np.float32)

    whole = g.Net(d)
    whole.set_weights(w0, b0)
    whole.set_data(x, y)
    libc_srand(31)
    whole.train_epochs(5)
    w_whole, b_whole = whole.get_weights()

    first = g.Net(d)
    first.set_weights(w0, b0)
    first.set_data(x, y)
    libc_srand(31)  # the resumed run continues the same rand() sequence: nothing else draws in between
    first.train_epochs(3)
    path = tmp_path / "net.state"
    first.save_state(path)
    first.close()

    second = g.Net(d)
    second.set_data(x, y)
    second.load_state(path)
    assert second.epochs() == 3
    second.train_epochs(2)
    w_res, b_res = second.get_weights()
    assert second.epochs() == whole.epochs() == 5
    assert np.array_equal(bits(w_res), bits(w_whole)) and np.array_equal(bits(b_res), bits(b_whole))
    if mode_name != "batched":
        # the open window's pending deltas came back too
        for k in range(3):
            assert np.array_equal(bits(second.pending_delta(k)), bits(whole.pending_delta(k)))
    whole.close()
    second.close()


def test_load_refuses_foreign_and_broken_files(g, tmp_path):
    if g.device_count() < 1:
        pytest.fail("no sm_100 device visible")
    d = g.make_desc([4, 5, 3], ["tanh", "sigmoid"], "regression", batch=4, lr=0.1, mode=g.MODE_BATCHED)
    net = g.Net(d)
    net.set_weights(np.zeros(g.weight_count(d), np.float32), None)
    path = tmp_path / "a.state"
    net.save_state(path)
    other = g.Net(g.make_desc([4, 6, 3], ["tanh", "sigmoid"], "regression", batch=4, lr=0.1, mode=g.MODE_BATCHED))
    with pytest.raises(RuntimeError):
        other.load_state(path)                       # another shape
    refm = g.Net(g.make_desc([4, 5, 3], ["tanh", "sigmoid"], "regression", batch=4, lr=0.1, mode=g.MODE_REFERENCE))
    with pytest.raises(RuntimeError):
        refm.load_state(path)                        # another arithmetic mode
    junk = tmp_path / "junk.state"
    junk.write_bytes(b"not a state file")
    with pytest.raises(RuntimeError):
        net.load_state(junk)
    cut = tmp_path / "cut.state"
    cut.write_bytes(path.read_bytes()[:-8])
    with pytest.raises(RuntimeError):
        net.load_state(cut)
    with pytest.raises(RuntimeError):
        net.load_state(tmp_path / "missing.state")
    for n in (net, other, refm):
        n.close()
