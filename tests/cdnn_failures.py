"""TEST INFRASTRUCTURE.  Failure paths of the B200 engine under NeoML, each made to happen on the host or by a wait
that is built to run out -- nothing here faults, traps or hangs a GPU.  Runs in a process of its own (see
tests/cdnn_parity.py) and prints one JSON line.

    python tests/cdnn_failures.py wait_timeout | memory_limit | free_while_pending | abort_distributed | padded_pool | ...
"""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from neoml_b200 import _capi, cdnn  # noqa: E402


def small_net(engine):
    rng = np.random.default_rng(5)
    f = rng.uniform(-1, 1, (16, 3, 3, 8)).astype(np.float32)
    b = rng.uniform(-1, 1, 16).astype(np.float32)
    x = rng.uniform(-1, 1, (2, 12, 12, 8)).astype(np.float32)
    net = cdnn.Net(engine, cdnn.Model.conv(f, b, padding=(1, 1)))
    net.set_input("in", x)
    return net


def wait_timeout():
    """A kernel's bounded wait runs out (20 ms limit, a barrier nothing completes): the status word is set, the engine
    reports it at the next device-to-host exchange and clears it, and the next pass is clean."""
    lib = _capi.load()
    engine = cdnn.Engine("gpu")
    net = small_net(engine)
    net.run()
    first = net.output("out")
    assert lib.nb200_device_status(None, 0) == 0
    assert lib.nb200_debug_wait_probe(None, 20_000_000) == 0
    status = lib.nb200_device_status(None, 0)           # reading synchronises the stream the probe ran on
    raised = ""
    try:
        net.run()
        net.output("out")
    except cdnn.CDnnError as exc:
        raised = str(exc)
    after = lib.nb200_device_status(None, 0)
    net.run()
    again = net.output("out")
    return {"status_after_probe": status, "raised": raised, "status_after_report": after,
            "clean_pass_matches": bool(np.array_equal(first, again)), "status_at_end": lib.nb200_device_status(None, 0)}


def memory_limit():
    """memoryLimit exceeded -> the exception handler's OnMemoryError (std::bad_alloc under NeoML's handler); an engine
    with room runs the same net."""
    small = cdnn.Engine("gpu", memory_limit=1 << 20)    # 1 MiB
    raised = ""
    try:
        rng = np.random.default_rng(6)
        net = cdnn.Net(small, cdnn.Model.conv(rng.uniform(-1, 1, (64, 3, 3, 64)).astype(np.float32), None, padding=(1, 1)))
        net.set_input("in", rng.uniform(-1, 1, (8, 56, 56, 64)).astype(np.float32))   # 6.4 MB: over the limit
        net.run()
    except cdnn.CDnnError as exc:
        raised = str(exc)
    small.close()
    roomy = cdnn.Engine("gpu", memory_limit=1 << 30)
    net = small_net(roomy)
    net.run()
    ok = bool(np.isfinite(net.output("out")).all())
    return {"raised": raised, "engine_with_room_runs": ok}


def filter_update():
    """The engine keeps a prepared form of every convolution filter; new filter values (here: a second model loaded
    into blobs that reuse the first one's memory, and a net whose filter is replaced by a fresh load) must be seen."""
    engine = cdnn.Engine("gpu")
    cpu = cdnn.Engine("cpu")
    rng = np.random.default_rng(9)
    x = rng.uniform(-1, 1, (8, 16, 16, 64)).astype(np.float32)     # 2048 output positions: the filter is prepared
    worst = 0.0
    for round_ in range(3):
        f = rng.uniform(-1, 1, (64, 3, 3, 64)).astype(np.float32)
        b = rng.uniform(-1, 1, 64).astype(np.float32)
        model = cdnn.Model.conv(f, b, padding=(1, 1))
        got_net, want_net = cdnn.Net(engine, model), cdnn.Net(cpu, model)
        for net in (got_net, want_net):
            net.set_input("in", x)
            net.run()
        for _ in range(2):                     # a second pass uses the kept form
            got_net.run()
        got, want = got_net.output("out"), want_net.output("out")
        worst = max(worst, float(np.abs(got - want).max() / np.sqrt(np.mean(want * want))))
        got_net.close()                        # frees the filter blob: the next round's may land on the same memory
        want_net.close()
        model.close()
    return {"worst_gate": worst}


def overlapped_input():
    """Six steps with six different batches through the double-buffered loop (the engine copies step i+1's batch while
    step i's kernels run) against the same batches fed one at a time: every step's result must be the same bits."""
    import torch
    from neoml_b200 import resnet50
    engine = cdnn.Engine("gpu")
    model = cdnn.Model.resnet50(resnet50.make_weights())
    net = cdnn.Net(engine, model)
    steps, batch, hw = 6, 8, 160                              # 2.4 MB per batch: above the engine's 1 MB threshold
    rng = np.random.default_rng(11)
    x = torch.from_numpy(rng.uniform(0, 1, (steps, batch, hw, hw, 3)).astype(np.float32)).pin_memory()
    per_out = batch * 1001
    out = torch.zeros(steps * per_out, dtype=torch.float32).pin_memory()
    net.set_input("in", x[0].numpy())
    net.time_steps(steps, "probs,argmax", source="in", input_ptr=x.data_ptr(), output_ptr=out.data_ptr(),
                   output_bytes=per_out * 4, double_buffered=True, input_stride_floats=x[0].numel(),
                   output_stride_bytes=per_out * 4)
    got = out.numpy().reshape(steps, per_out).copy()
    same = True
    for i in range(steps):
        net.set_input("in", x[i].numpy())
        net.run()
        want = np.concatenate([net.output("probs").ravel(), net.output("argmax").ravel().view(np.float32)])
        same = same and bool(np.array_equal(got[i].view(np.int32), want.view(np.int32)))
    return {"all_steps_bit_identical": same}


def free_while_pending():
    engine = cdnn.Engine("gpu")
    return {"max_difference": cdnn.selftest_free_while_pending(engine)}


def padded_pool():
    """BlobResizeImage + BlobMaxPooling in every order of touching the buffers (see cdnn_selftest_padded_pool); the same
    harness on the reference CPU engine is the control."""
    engine = cdnn.Engine("gpu")
    wrong, launches = cdnn.selftest_padded_pool(engine)
    return {"mismatches": wrong, "launches_pad_plus_pool": launches}


def attention_chain():
    """The attention score chain in every order of touching its buffers (see cdnn_selftest_attention_chain)."""
    engine = cdnn.Engine("gpu")
    worst, launches = cdnn.selftest_attention_chain(engine)
    return {"worst_error": worst, "launches_of_the_chain": launches}


def normalization_chain():
    """The object-normalisation chains in every order of touching their buffers (cdnn_selftest_normalization_chain)."""
    engine = cdnn.Engine("gpu")
    worst, launches = cdnn.selftest_normalization_chain(engine)
    return {"worst_error": worst, "launches_of_the_output_chain": launches}


def product_chain():
    """A fully connected product with bias, GELU gate or residual sum in every order of touching the buffers."""
    engine = cdnn.Engine("gpu")
    return {"worst_error": cdnn.selftest_product_chain(engine)}


def _state_gap(got, want):
    """Largest difference in any buffer of a random program's final state, relative to that buffer's largest value
    (at least 1): a product of large operands that cancels to a small sum is judged by the size of what was summed."""
    size = 24 * 32
    pieces = [slice(i * size, (i + 1) * size) for i in range(6)] + [slice(6 * size, got.size)]
    gap = 0.0
    for piece in pieces:
        diff = float(np.max(np.abs(got[piece] - want[piece])))
        scale = max(1.0, float(np.max(np.abs(want[piece]))))
        if not np.isfinite(diff) or not np.isfinite(scale):
            return 1e30
        gap = max(gap, diff / scale)
    return gap


def random_program():
    """Seeded random programs of the calls the engine holds back, notes or fuses, on the B200 engine and on the reference
    CPU engine (the control): the buffers must end in the same state."""
    gpu, cpu = cdnn.Engine("gpu"), cdnn.Engine("cpu")
    worst, worst_seed = 0.0, -1
    # the second range holds the programs that once caught a copy of an in-place note reading its source too late
    # and the third one (seeds from 1 000 000 on also draw whole layer chains, cut short at random) those that caught a
    # note written, when touched, ahead of a call recorded before it
    programs = ([(1000 + i, 20 + 7 * (i % 9)) for i in range(40)] + [(5000 + i, 15 + 11 * (i % 13)) for i in range(600)]
                + [(1000000 + i, 15 + 11 * (i % 13)) for i in range(2000)]
                # from 2 000 000 on: also statistics in a stack variable and blobs that die while a note still reads them
                + [(2000000 + i, 15 + 11 * (i % 13)) for i in range(2000)]
                # from 3 000 000 on: also the calls of attention (scores, scale, mask, softmax, values) in any order
                + [(3000000 + i, 15 + 11 * (i % 13)) for i in range(1200)]
                # from 4 000 000 on: also convolutions with their in-place sum and ReLU, filters rewritten, sources released
                + [(4000000 + i, 15 + 11 * (i % 13)) for i in range(1500)]
                # from 5 000 000 on: 1024-row matrices (an engine may keep a prepared form of a product's weights), the
                # weights also written on the device and reallocated
                + [(5000000 + i, 15 + 11 * (i % 13)) for i in range(1000)]
                # from 6 000 000 on: small matrices, everything above, and a stem's border + pooling around the convolutions
                + [(6000000 + i, 15 + 11 * (i % 13)) for i in range(1500)])
    for seed, steps in programs:
        got = cdnn.selftest_random_program(gpu, seed, steps)
        want = cdnn.selftest_random_program(cpu, seed, steps)
        gap = _state_gap(got, want)
        if gap > worst:
            worst, worst_seed = gap, seed
    return {"worst_gap": worst, "seed": worst_seed}


def random_program_cpu():
    """The random programs themselves, on the reference CPU engine alone (no GPU needed): every class of seeds runs,
    gives finite values, and gives the same values when it runs again (a program must depend on its seed only)."""
    cpu = cdnn.Engine("cpu")
    classes, worst = {}, 0.0
    for base in (1000, 5000, 1000000, 2000000, 3000000, 4000000, 5000000, 6000000):
        for i in range(12):
            steps = 15 + 11 * (i % 13)
            first = cdnn.selftest_random_program(cpu, base + i, steps)
            again = cdnn.selftest_random_program(cpu, base + i, steps)
            ok = bool(np.isfinite(first).all() and np.array_equal(first, again))
            classes[str(base)] = classes.get(str(base), True) and ok
            worst = max(worst, float(np.max(np.abs(first))))
        other = cdnn.selftest_random_program(cpu, base + 1, 15 + 11)
        classes[str(base)] = classes[str(base)] and not np.array_equal(other, cdnn.selftest_random_program(cpu, base + 2, 15 + 11))
    return {"classes": classes, "largest_value": worst}


def launch_counts():
    """Kernel launches per CDnn::RunOnce: what the engine's run-time fusion leaves of the call sequences NeoML issues.
    ResNet-50 makes 106 BlobConvolution + 130 element-wise / pooling / resize calls per pass, an encoder layer about 60
    calls; the counts below are what is launched for them."""
    from neoml_b200 import resnet50
    lib = _capi.load()
    engine = cdnn.Engine("gpu")
    rng = np.random.default_rng(21)
    out = {}
    net = cdnn.Net(engine, cdnn.Model.resnet50(resnet50.make_weights()))
    net.set_input("in", rng.uniform(0, 1, (32, 224, 224, 3)).astype(np.float32))
    net.run()
    before = lib.nb200_launch_count()
    net.run()
    out["resnet50_launches_per_pass"] = int(lib.nb200_launch_count() - before)
    net.close()
    layers, heads, seq = 2, 2, 128
    net = cdnn.Net(engine, cdnn.Model.transformer(layers, 64 * heads, heads, 256, seed=3, sigma=0.05, mask=True))
    net.set_input("in", rng.standard_normal((4, seq, 64 * heads)).astype(np.float32))
    net.set_input("mask", np.triu(np.ones((seq, seq), np.float32), 1), (1, 1, 1, 1, seq, 1, seq))
    net.run()
    before = lib.nb200_launch_count()
    net.run()
    out["transformer_launches_per_layer"] = (lib.nb200_launch_count() - before) / layers
    return out


def abort_distributed():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    cdnn.load()
    return {"raised": cdnn.selftest_abort_distributed((0, 1))}


if __name__ == "__main__":
    print(json.dumps({"case": sys.argv[1], **globals()[sys.argv[1]]()}))
