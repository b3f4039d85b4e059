"""Failure paths of the engine under NeoML (tests/cdnn_failures.py, one process per case): a bounded device wait that
runs out, the memory limit, a blob freed while the call that reads it is still recorded, AbortDistributed.
No case faults, traps or hangs a GPU: waits are built to expire after 20 ms, the abort happens between steps."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def run_case(name: str) -> dict:
    if not (ROOT / "neoml_b200" / "lib" / "host" / "libcdnn_host.so").exists():
        pytest.skip("hosted NeoML libraries not built")
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "cdnn_failures.py"), name], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, f"{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_bounded_wait_that_runs_out_is_reported_and_the_engine_stays_usable():
    row = run_case("wait_timeout")
    assert row["status_after_probe"] == 0x7E01
    assert "bounded-wait timeout" in row["raised"]
    assert row["status_after_report"] == 0 and row["status_at_end"] == 0
    assert row["clean_pass_matches"]


def test_memory_limit_raises_the_memory_error():
    row = run_case("memory_limit")
    assert "bad_alloc" in row["raised"], row
    assert row["engine_with_room_runs"]


def test_source_freed_while_the_convolution_is_still_recorded():
    assert run_case("free_while_pending")["max_difference"] == 0.0


def test_abort_distributed_ends_the_peers_next_collective():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    row = run_case("abort_distributed")
    assert "Stopping due to error in another thread." in row["raised"]


def test_prepared_filters_follow_new_filter_values():
    assert run_case("filter_update")["worst_gate"] < 1e-4


def test_input_copies_that_overlap_the_previous_step_change_nothing():
    assert run_case("overlapped_input")["all_steps_bit_identical"]


def test_padding_that_is_only_noted_is_never_observable():
    """The engine pools the unpadded image in one pass and leaves the padded image unwritten until somebody looks."""
    row = run_case("padded_pool")
    assert row["mismatches"] == 0
    assert row["launches_pad_plus_pool"] == 1


def test_attention_scores_that_are_only_noted_are_never_observable():
    """The engine runs the five calls of the chain as one kernel and writes scores and probabilities only for whoever
    reads them; early releases and an overwritten input change nothing."""
    row = run_case("attention_chain")
    assert row["worst_error"] < 1e-4, row
    assert row["launches_of_the_chain"] == 1


def test_normalisation_steps_that_are_only_noted_are_never_observable():
    """Shift, square, row sums as one pass; shift, row scale, column scale, column shift as one pass (same roundings as
    the separate calls); an overwritten or released row vector changes nothing."""
    row = run_case("normalization_chain")
    assert row["worst_error"] == 0.0, row
    assert row["launches_of_the_output_chain"] == 1


def test_fully_connected_products_that_are_only_noted_are_never_observable():
    """Bias, residual sum and the GELU gate ride in the product's epilogue; reading the plain product afterwards,
    a gate noted in part and overwritten weights all give what the separate calls give."""
    assert run_case("product_chain")["worst_error"] < 5e-5


def test_random_programs_end_in_the_state_the_reference_engine_ends_in():
    """9 840 random call sequences (in place or not, shared allocations, buffers released in the middle, weights
    replaced, whole layer chains cut short, temporaries that die early, the calls of attention and those around a convolution in any order) leave every buffer as the reference CPU engine leaves it: nothing the engine
    holds back is observable.  The gap is the largest difference in a buffer over that buffer's largest value (at least 1).
    Rounding alone separates the engines by up to 2.6e-4 (worst of 29 640 programs; a long program amplifies it); one call
    carried out twice, too late or too early shows as 1e-3 to 10."""
    row = run_case("random_program")
    assert row["worst_gap"] < 5e-4, row


def test_the_fusions_hold_in_a_cdnn():
    """A regression in the engine's run-time fusion would still give right results, only slower: pin the launch counts.
    ResNet-50: 54 contractions + stem padding + ONE pooling pass + five small kernels (no separate add, ReLU, resize or
    per-pass filter preparation).  Encoder layer: six products, one attention kernel, four transposes, and per
    normalisation two row-sum passes, five vector-sized launches and one normalise-scale-shift pass."""
    row = run_case("launch_counts")
    assert row["resnet50_launches_per_pass"] <= 80, row     # 61 at batch 256; small batches add split-K finishing passes
    assert row["transformer_launches_per_layer"] <= 42, row  # 34 at full size; about 60 calls arrive
