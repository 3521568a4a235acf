"""Small file helpers: atomic writes and media encoding.

``atomic_put`` writes to a temporary sibling, fsyncs and renames, so a reader never sees
a half-written file (checkpoint pointers, configs, sample artifacts).

Parity: reference ``wm/infra/io.py:27-91``.
"""

from __future__ import annotations

import os
import tempfile
from io import BytesIO
from typing import Any

import numpy as np

PathLike = str | os.PathLike

__all__ = [
    "atomic_put",
    "atomic_put_text",
    "encode_image",
    "encode_video",
    "exists",
    "get",
    "get_text",
    "join_path",
]


def join_path(root: PathLike, *parts: PathLike) -> str:
    return os.path.join(os.fspath(root), *(os.fspath(p) for p in parts))


def exists(path: PathLike) -> bool:
    return os.path.exists(path)


def get(path: PathLike) -> bytes:
    with open(path, "rb") as handle:
        return handle.read()


def get_text(path: PathLike, encoding: str = "utf-8") -> str:
    return get(path).decode(encoding)


def atomic_put(payload: bytes | BytesIO, path: PathLike) -> None:
    data = payload.getvalue() if isinstance(payload, BytesIO) else bytes(payload)
    path = os.fspath(path)
    directory = os.path.dirname(path) or "."
    os.makedirs(directory, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=".tmp-", dir=directory)
    try:
        with os.fdopen(fd, "wb") as handle:
            handle.write(data)
            handle.flush()
            os.fsync(handle.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def atomic_put_text(text: str, path: PathLike, encoding: str = "utf-8") -> None:
    atomic_put(text.encode(encoding), path)


def encode_image(pixels: np.ndarray, *, file_format: str, **options: Any) -> BytesIO:
    """Encode an ``[H, W, 3]`` uint8 array with Pillow."""
    from PIL import Image

    buffer = BytesIO()
    name = "JPEG" if file_format.lower() in ("jpg", "jpeg") else file_format.upper()  # Pillow's names
    Image.fromarray(np.ascontiguousarray(pixels)).save(buffer, format=name, **options)
    buffer.seek(0)
    return buffer


def _encode_with_opencv(pixels: np.ndarray, fps: int) -> bytes | None:
    """mp4 bytes written by OpenCV into a scratch file, or ``None`` when that is not possible."""
    try:
        import cv2
    except ImportError:
        return None
    import tempfile

    height, width = int(pixels.shape[1]), int(pixels.shape[2])
    with tempfile.TemporaryDirectory() as scratch:
        target = os.path.join(scratch, "clip.mp4")
        writer = cv2.VideoWriter(target, cv2.VideoWriter_fourcc(*"mp4v"), float(max(fps, 1)), (width, height))
        if not writer.isOpened():
            return None
        try:
            for frame in pixels:
                writer.write(cv2.cvtColor(np.ascontiguousarray(frame), cv2.COLOR_RGB2BGR))
        finally:
            writer.release()
        try:
            with open(target, "rb") as handle:
                data = handle.read()
        except OSError:
            return None
    return data or None


def encode_video(pixels: np.ndarray, *, fps: int, quality: int = 8) -> BytesIO:
    """Encode ``[T, H, W, 3]`` uint8 frames.

    mp4 through ``imageio`` with the ffmpeg plugin, else through OpenCV's ``mp4v`` encoder;
    with neither, the frames are stored as an animated GIF through Pillow so that sampling
    never kills training.
    """
    buffer = BytesIO()
    try:
        import imageio.v2 as imageio  # type: ignore

        with imageio.get_writer(buffer, format="mp4", fps=fps, quality=quality) as writer:
            for frame in pixels:
                writer.append_data(frame)
    except ImportError:
        encoded = _encode_with_opencv(pixels, fps)
        if encoded is not None:
            return BytesIO(encoded)
        from PIL import Image

        frames = [Image.fromarray(np.ascontiguousarray(f)) for f in pixels]
        frames[0].save(
            buffer,
            format="GIF",
            save_all=True,
            append_images=frames[1:],
            duration=max(1, int(1000 / max(fps, 1))),
            loop=0,
        )
    buffer.seek(0)
    return buffer
