"""SHA-256 manifest of a checkpoint directory and a cached verification receipt.

``manifest.sha256`` holds ``sha256sum``-style rows (index first, then the other files in
lexical order); the checkpoint fingerprint reported in every reply is the SHA-256 of those
rows.  Verification hashes each file once and caches a receipt keyed by size and mtime so a
later start only re-hashes files that changed.  Parity: engine/crates/model/src/flash/
manifest.rs:22-29,194-397; engine/crates/hash/src/lib.rs:13-40 (streaming digest).
"""
from __future__ import annotations

import hashlib
import json
import os

MANIFEST = "manifest.sha256"
RECEIPT = ".manifest.receipt.json"
_CHUNK = 8 << 20


def digest_file(path: str) -> str:
    """Streaming SHA-256 of a file: the native reader (csrc/host/host_runtime.cpp) for anything large, hashlib otherwise."""
    if os.path.getsize(path) >= (1 << 20):
        from ..utils.native import host
        m = host()
        if m is not None:
            return m.sha256_file(path)[0]
    h = hashlib.sha256()
    with open(path, "rb", buffering=0) as f:
        while True:
            b = f.read(_CHUNK)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def _files(root: str) -> list:
    names = [n for n in sorted(os.listdir(root))
             if os.path.isfile(os.path.join(root, n)) and n not in (MANIFEST, RECEIPT) and not n.endswith(".tmp")]
    idx = "model.safetensors.index.json"
    if idx in names:
        names.remove(idx)
        names.insert(0, idx)
    return names


def write_manifest(root: str) -> str:
    rows = [f"{digest_file(os.path.join(root, n))}  {n}\n" for n in _files(root)]
    with open(os.path.join(root, MANIFEST), "w") as f:
        f.writelines(rows)
    return fingerprint(root)


def fingerprint(root: str) -> str:
    with open(os.path.join(root, MANIFEST), "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


class ManifestError(ValueError):
    pass


def verify(root: str, use_receipt: bool = True) -> dict:
    """Check every manifest row; returns {"fingerprint", "files", "hashed", "cached"}."""
    mpath = os.path.join(root, MANIFEST)
    if not os.path.exists(mpath):
        raise ManifestError(f"{root}: no {MANIFEST}")
    rows = {}
    with open(mpath) as f:
        for line in f:
            if not line.strip():
                continue
            try:
                digest, name = line.rstrip("\n").split("  ", 1)
            except ValueError:
                raise ManifestError(f"malformed manifest row {line!r}") from None
            if "/" in name or name.startswith("."):
                raise ManifestError(f"manifest names a file outside the directory: {name!r}")
            rows[name] = digest
    receipt = {}
    rpath = os.path.join(root, RECEIPT)
    if use_receipt and os.path.exists(rpath):
        try:
            with open(rpath) as f:
                receipt = json.load(f)
        except ValueError:
            receipt = {}
    hashed = cached = 0
    new_receipt = {}
    for name, digest in rows.items():
        path = os.path.join(root, name)
        if not os.path.exists(path):
            raise ManifestError(f"{name}: listed in the manifest but missing")
        stt = os.stat(path)
        key = [stt.st_size, stt.st_mtime_ns, digest]
        if receipt.get(name) == key:
            cached += 1
        else:
            got = digest_file(path)
            hashed += 1
            if got != digest:
                raise ManifestError(f"{name}: sha256 {got} does not match the manifest")
        new_receipt[name] = key
    extra = set(n for n in _files(root) if n.endswith(".safetensors")) - set(rows)
    if extra:
        raise ManifestError(f"weight files not covered by the manifest: {sorted(extra)}")
    try:
        tmp = rpath + ".tmp"
        with open(tmp, "w") as f:
            json.dump(new_receipt, f)
        os.replace(tmp, rpath)
    except OSError:
        pass
    return {"fingerprint": fingerprint(root), "files": len(rows), "hashed": hashed, "cached": cached}
