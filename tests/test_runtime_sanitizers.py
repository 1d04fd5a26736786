"""The native runtime (dependency engine, storage pools) under ThreadSanitizer and AddressSanitizer + UBSan: the C++
stress test is compiled together with the runtime sources and run as an executable; a data race, a leak of a freed
block or undefined behaviour makes the sanitizer print a report and exit non-zero."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCES = [os.path.join(ROOT, 'cpp-package', 'tests', 'runtime_stress.cc'), os.path.join(ROOT, 'mxnet_b200', 'csrc', 'engine.cc'),
           os.path.join(ROOT, 'mxnet_b200', 'csrc', 'storage.cc')]


def _build(tmp_path, flags):
    exe = str(tmp_path / 'runtime_stress')
    r = subprocess.run(['g++', '-std=c++17', '-g', '-O1', '-pthread'] + flags + SOURCES + ['-ldl', '-lrt', '-o', exe],
                       capture_output=True, text=True)
    if r.returncode != 0 and ('sanitizer' in r.stderr or 'cannot find -l' in r.stderr):
        pytest.skip('sanitizer runtime not installed: %s' % r.stderr.strip().splitlines()[-1])
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


@pytest.mark.skipif(shutil.which('g++') is None, reason='needs a C++ compiler')
@pytest.mark.parametrize('name,flags,env', [
    ('plain', [], {}),
    ('thread', ['-fsanitize=thread'], {'TSAN_OPTIONS': 'halt_on_error=1 exitcode=66'}),
    ('address+undefined', ['-fsanitize=address,undefined', '-fno-omit-frame-pointer', '-fno-sanitize-recover=undefined'],
     {'ASAN_OPTIONS': 'detect_leaks=1 exitcode=67'}),
])
def test_runtime_stress_under_sanitizer(tmp_path, name, flags, env):
    exe = _build(tmp_path, flags)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=dict(os.environ, **env))
    assert r.returncode == 0, '%s build: exit %d\n%s\n%s' % (name, r.returncode, r.stdout[-2000:], r.stderr[-4000:])
    assert 'all checks passed' in r.stdout
    assert 'WARNING: ThreadSanitizer' not in r.stderr and 'ERROR: AddressSanitizer' not in r.stderr
    assert 'runtime error:' not in r.stderr
