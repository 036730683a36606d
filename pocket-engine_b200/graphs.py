"""Captured graph sets for decode steps with adapters (src/engine.rs:164-166, 437-471, 698-721): one CUDA graph
per batch bucket, each holding the step's grouping kernel and the block's adapter kernels with ``max_tiles`` and
``rows`` equal to the bucket. A step picks the smallest bucket that holds its sequences, uploads its tile words
and replays; moving adapters between GPU slots only changes slabs and descriptor tables the kernels read, so no
graph is captured again (docs/design.md:84 of the engine). torch supplies the capture; the kernels are the
library's."""

BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 160, 192, 224, 256)


class LoraGraphSet:
    def __init__(self, loras, body, max_seqs, stream, buckets=BUCKETS):
        """``body(step, rows, stream_handle)`` issues the block's layers (Linear.forward with lora=step) on buffers
        that stay where they are; ``stream`` is the torch stream steps will run on."""
        import numpy as np
        import torch
        self.loras, self.stream = loras, stream
        self.graphs = {}
        s = stream.cuda_stream
        empty = np.zeros(1, np.int32)  # zero tiles
        with torch.cuda.stream(stream):
            for b in buckets:
                if b > max_seqs:
                    break
                loras.meta_upload(empty, s)
                body(loras.lora_step(b, s, decode=True), b, s)  # a plain run first, outside capture
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    body(loras.lora_step(b, s, decode=True), b, s)
                self.graphs[b] = g
        stream.synchronize()

    def bucket(self, n_seqs):
        for b in sorted(self.graphs):
            if b >= n_seqs:
                return b
        return None

    def replay(self, n_seqs, tile_words):
        """One decode step of ``n_seqs`` one-token sequences; returns the bucket used. The caller has already put
        the step's activations into the captured buffers and queued any slot uploads on the same stream."""
        import torch
        b = self.bucket(n_seqs)
        if b is None:
            raise ValueError(f"{n_seqs} sequences exceed the largest captured bucket")
        with torch.cuda.stream(self.stream):
            self.loras.meta_upload(tile_words, self.stream.cuda_stream)
            self.graphs[b].replay()
        return b
