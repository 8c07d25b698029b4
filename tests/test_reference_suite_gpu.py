"""The reference's own hard-path tests, unmodified, against the drop-in `cu_flash_dism`.

The reference's Python wrappers (dism_v3/python/flash_dism/{summary,hard_forward,hard_backward,varlen}.py and its
FP64 oracle reference/dism_v3_ref.py) are linked by path into a scratch package next to this library's
`cu_flash_dism`, and pytest runs dism_v3/tests/test_hard_{summary,chunk,forward,backward}.py in a child process.
Left out: the `codegen` cases (they disassemble the reference's object files) and the sanitizer smoke test.  Every
other case has to pass, the CUDA-graph capture and replay cases included.  Needs a reference checkout
(the REFERENCE_ROOT environment variable, or the default below); without one the test is skipped.
"""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_ROOT = os.environ.get('REFERENCE_ROOT', '/root/reference')
MODULES = ('summary.py', 'hard_forward.py', 'hard_backward.py', 'varlen.py', os.path.join('reference', 'dism_v3_ref.py'))
TESTS = ('test_hard_summary.py', 'test_hard_chunk.py', 'test_hard_forward.py', 'test_hard_backward.py')
LEFT_OUT = 'not codegen and not sanitizer'


def test_reference_hard_tests_pass_against_the_dropin(tmp_path):
    package = os.path.join(REFERENCE_ROOT, 'dism_v3', 'python', 'flash_dism')
    tests = os.path.join(REFERENCE_ROOT, 'dism_v3', 'tests')
    if not all(os.path.exists(os.path.join(package, m)) for m in MODULES) or not all(os.path.exists(os.path.join(tests, t)) for t in TESTS):
        pytest.skip(f'no reference checkout under {REFERENCE_ROOT}')
    scratch = tmp_path / 'flash_dism'
    (scratch / 'reference').mkdir(parents=True)
    (scratch / '__init__.py').write_text('')
    (scratch / 'reference' / '__init__.py').write_text('')
    for module in MODULES:
        os.symlink(os.path.join(package, module), scratch / module)
    import dism_b200
    # the scratch package first (its flash_dism is the reference's), then the drop-in directory (for cu_flash_dism)
    environment = dict(os.environ, PYTHONPATH=os.pathsep.join([str(tmp_path), dism_b200.DROPIN_PATH, ROOT]), PYTHONDONTWRITEBYTECODE='1')
    command = [sys.executable, '-m', 'pytest', '-q', '-p', 'no:cacheprovider', '-rA', '-k', LEFT_OUT, *TESTS]
    result = subprocess.run(command, cwd=tests, env=environment, capture_output=True, text=True, timeout=1500)
    outcomes = {case: outcome for outcome, case in re.findall(r'^(PASSED|FAILED|ERROR) (\S+)', result.stdout, re.M)}
    assert outcomes, result.stdout[-3000:] + result.stderr[-3000:]
    unexpected = sorted(case for case, outcome in outcomes.items() if outcome != 'PASSED')
    print(f"{sum(o == 'PASSED' for o in outcomes.values())} of {len(outcomes)} reference cases passed")
    assert not unexpected, 'reference cases failed against the drop-in:\n' + '\n'.join(unexpected) + '\n' + result.stdout[-6000:]
