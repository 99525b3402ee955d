"""SHA-256 checksum of an archive file and its sidecar (reference: pybuda/pybuda/tti/utils.py)."""
import hashlib
import os


def compute_file_checksum(file_path, chunk_size=1 << 20):
    h = hashlib.sha256()
    with open(file_path, "rb") as f:
        for chunk in iter(lambda: f.read(chunk_size), b""):
            h.update(chunk)
    return h.hexdigest()


def write_checksum_to_file(checksum, output_file_path):
    with open(output_file_path, "w") as f:
        f.write(checksum)


def read_checksum_from_file(checksum_file_name):
    """The stored checksum, or None when there is no sidecar file."""
    if not os.path.exists(checksum_file_name):
        return None
    with open(checksum_file_name, "r") as f:
        return f.read().strip()
