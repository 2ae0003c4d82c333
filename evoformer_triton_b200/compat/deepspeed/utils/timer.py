"""``SynchronizedWallClockTimer.memory_usage`` as used by memory_benchmark.py:38."""
import torch


class SynchronizedWallClockTimer:
    @staticmethod
    def memory_usage() -> str:
        gb = 1024.0 ** 3
        return (f" | mem_allocated: {torch.cuda.memory_allocated() / gb:.4f} GB"
                f" | max_mem_allocated: {torch.cuda.max_memory_allocated() / gb:.4f} GB"
                f" | cache_allocated: {torch.cuda.memory_reserved() / gb:.4f} GB"
                f" | max_cache_allocated: {torch.cuda.max_memory_reserved() / gb:.4f} GB")
