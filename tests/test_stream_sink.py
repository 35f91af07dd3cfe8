"""The stream output: local files appear only when complete; under a gcsfuse mount the bytes go to the bucket through the
storage client (a fake here), never through the mount."""
import os

import numpy as np
import pytest

from util import ROOT  # noqa: F401
from dttt_b200.data import prep


class FakeBlob:
    def __init__(self, store, name):
        self.store, self.name, self.bucket = store, name, None

    def exists(self):
        return self.name in self.store

    def open(self, mode, chunk_size=None, ignore_flush=None):
        import io
        blob = self

        class W(io.BytesIO):
            def close(self_inner):
                blob.store[blob.name] = self_inner.getvalue()
                super().close()
        return W()

    def rewrite(self, src, token=None):
        # two rounds, to exercise the continuation token
        if token is None and len(src.store[src.name]) > 8:
            return "more", 0, 0
        self.store[self.name] = src.store[src.name]
        return None, 0, 0

    def delete(self):
        del self.store[self.name]


class FakeClient:
    def __init__(self):
        self.objects = {}

    def bucket(self, name):
        client = self

        class B:
            def blob(self, obj):
                return FakeBlob(client.objects.setdefault(name, {}), obj)
        return B()


def test_bucket_object_picks_the_deepest_gcsfuse_mount(tmp_path):
    mounts = tmp_path / "mounts"
    mounts.write_text("proc /proc proc rw 0 0\nmybucket /mnt/b fuse rw 0 0\nother /mnt/b/deep fuse rw 0 0\n/dev/sda1 /mnt/c fuse rw 0 0\n")
    assert prep.bucket_object("/mnt/b/x/tokens.u32", str(mounts)) == ("mybucket", "x/tokens.u32")
    assert prep.bucket_object("/mnt/b/deep/y", str(mounts)) == ("other", "y")
    assert prep.bucket_object("/mnt/c/y", str(mounts)) is None            # a device, not a bucket
    assert prep.bucket_object("/home/y", str(mounts)) is None


def test_sink_uploads_under_a_mount_and_renames_at_the_end(tmp_path):
    mounts = tmp_path / "mounts"
    mounts.write_text("bkt /gcs fuse rw 0 0\n")
    client = FakeClient()
    sink = prep.StreamSink("/gcs/data/a/tokens.u32", client=client, mounts_file=str(mounts))
    assert not sink.exists()
    with sink:
        sink.write(np.arange(5, dtype=np.uint32))
        assert "data/a/tokens.u32" not in client.objects["bkt"]          # nothing under the final name yet
    assert sink.exists() and sink.bytes == 20
    assert np.frombuffer(client.objects["bkt"]["data/a/tokens.u32"], dtype="<u4").tolist() == [0, 1, 2, 3, 4]
    assert "data/a/tokens.u32.tmp" not in client.objects["bkt"]
    with pytest.raises(RuntimeError):
        with prep.StreamSink("/gcs/data/b", client=client, mounts_file=str(mounts)) as s2:
            s2.write(b"partial")
            raise RuntimeError("stop")
    assert "data/b" not in client.objects["bkt"] and "data/b.tmp" not in client.objects["bkt"]


def test_local_sink_leaves_no_partial_file(tmp_path):
    p = str(tmp_path / "d" / "x.bin")
    with pytest.raises(ValueError):
        with prep.StreamSink(p) as s:
            s.write(b"abc")
            raise ValueError
    assert not os.path.exists(p) and not os.path.exists(p + ".tmp")
    with prep.StreamSink(p) as s:
        s.write(b"abc")
    assert open(p, "rb").read() == b"abc"
