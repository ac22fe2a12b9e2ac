"""Install an unmodified copy of the reference package under oracle/_ref (TEST AND BENCHMARK INFRASTRUCTURE).

    python oracle/make_ref.py [path of a reference checkout]

The path defaults to the environment variable VESTA_REFERENCE, then to a directory named `reference` next to this
repository. The checkout is copied to a temporary directory (its own tree may be read-only and the build writes
into it) and installed with pip, offline and without dependencies, into oracle/_ref, which is git-ignored: no file
of the reference enters this repository's history. What uses the copy:
  * bench.py --impl reference and the cpu_baseline leg time its vesta/interp.py (the reference's CPU implementation
    of the decode step) on the host cores;
  * bench.py's ref_kernel block runs its generated GPU kernel through its own VestaGPT2.step path;
  * vesta/interp.py of this repository's drop-in package forwards `run` to it.
Nothing on the product's step path imports it.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
DEST = os.path.join(HERE, '_ref')


def find_checkout(path=None):
    for cand in (path, os.environ.get('VESTA_REFERENCE'), os.path.join(os.path.dirname(ROOT), 'reference')):
        if cand and os.path.exists(os.path.join(cand, 'vesta', 'interp.py')):
            return os.path.abspath(cand)
    return None


def install(path=None, quiet=True):
    """-> the installed directory, or None when no checkout is available (an existing copy is kept)"""
    src = find_checkout(path)
    if src is None:
        return DEST if os.path.exists(os.path.join(DEST, 'vesta', 'interp.py')) else None
    with tempfile.TemporaryDirectory() as tmp:
        work = os.path.join(tmp, 'reference')
        shutil.copytree(src, work, ignore=shutil.ignore_patterns('.git', '__pycache__'))
        if os.path.exists(DEST):
            shutil.rmtree(DEST)
        cmd = [sys.executable, '-m', 'pip', 'install', '--no-index', '--no-build-isolation', '--no-deps', '--target', DEST, work]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError('pip could not install the reference checkout:\n' + r.stdout[-2000:] + r.stderr[-2000:])
        if not quiet:
            print(r.stdout[-500:])
    return DEST


if __name__ == '__main__':
    d = install(sys.argv[1] if len(sys.argv) > 1 else None, quiet=False)
    print('installed under' if d else 'no reference checkout found:', d or 'pass its path or set VESTA_REFERENCE')
