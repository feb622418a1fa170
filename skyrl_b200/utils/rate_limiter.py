"""Async rate limiting for trajectory submission: a token bucket (requests per second with burst) combined
with a concurrency cap (reference: skyrl/train/utils/rate_limiter.py)."""

from __future__ import annotations

import asyncio
import time
from typing import Optional


class TokenBucket:
    def __init__(self, rate_per_s: float, burst: Optional[float] = None):
        if rate_per_s <= 0:
            raise ValueError("rate_per_s must be positive")
        self.rate = float(rate_per_s)
        self.capacity = float(burst if burst is not None else max(1.0, rate_per_s))
        self.tokens = self.capacity
        self.stamp = time.monotonic()
        self._lock = asyncio.Lock()

    def _refill(self) -> None:
        now = time.monotonic()
        self.tokens = min(self.capacity, self.tokens + (now - self.stamp) * self.rate)
        self.stamp = now

    async def acquire(self, n: float = 1.0) -> None:
        if n > self.capacity:
            raise ValueError(f"cannot acquire {n} tokens from a bucket of capacity {self.capacity}")
        while True:
            async with self._lock:
                self._refill()
                if self.tokens >= n:
                    self.tokens -= n
                    return
                wait = (n - self.tokens) / self.rate
            await asyncio.sleep(wait)


class RateLimiter:
    """``async with limiter:`` bounds both the start rate and the number of in-flight operations."""

    def __init__(self, rate_per_s: Optional[float] = None, max_concurrency: Optional[int] = None, burst: Optional[float] = None):
        self.bucket = TokenBucket(rate_per_s, burst) if rate_per_s else None
        self.sem = asyncio.Semaphore(max_concurrency) if max_concurrency else None
        self.in_flight = 0
        self.started = 0

    async def __aenter__(self):
        if self.sem is not None:
            await self.sem.acquire()
        try:
            if self.bucket is not None:
                await self.bucket.acquire()
        except BaseException:
            if self.sem is not None:
                self.sem.release()
            raise
        self.in_flight += 1
        self.started += 1
        return self

    async def __aexit__(self, *exc):
        self.in_flight -= 1
        if self.sem is not None:
            self.sem.release()
        return False
