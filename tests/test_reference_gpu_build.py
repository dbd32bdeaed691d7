"""The reference's own GPU path (its fp32 CUDA kernels + cuBLAS, compiled unmodified for sm_100a into oracle/_ref/cuda) as a
second checker: on the same seeded BERT-base weights and inputs this library's fp32 path must agree with it to the fp32
tolerance of the model tests (1e-3 max-abs on final hidden states), and the fp16 path to the fp16 tolerance (2e-2).

The comparison runs in a worker process (tests/ref_gpu_worker.py) because the reference's CPU and GPU builds cannot be
imported together; the worker also times both, and the test prints those times (run with -s to see them).
"""
import json
import os
import subprocess
import sys

import pytest

from oracle import ref_driver

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not ref_driver.cuda_build_available(), reason="oracle/_ref/cuda is not built (python oracle/build_ref.py --cuda)")
def test_fp32_and_fp16_paths_agree_with_the_reference_gpu_path():
    r = subprocess.run([sys.executable, os.path.join(HERE, "ref_gpu_worker.py"), "--layers", "12", "--iters", "6"],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("REF_GPU_RESULT ")][-1]
    res = json.loads(line[len("REF_GPU_RESULT "):])
    print(json.dumps(res, indent=1))
    for case in ("b1_s128", "b20_s128"):
        assert res[case]["seq_maxdiff"] < 1e-3 and res[case]["pooled_maxdiff"] < 1e-3, res[case]
    assert res["varlen_b64"]["seq_maxdiff"] < 1e-3, res["varlen_b64"]
    assert res["varlen_b64"]["fp16_seq_maxdiff"] < 2e-2, res["varlen_b64"]
