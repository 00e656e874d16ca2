"""Spectra with the tensor FFT methods: a two-tone signal, windowing against leakage, round trip, convolution theorem."""
import _path  # noqa: F401
import math

import torch

import rustorch as rt

n, fs = 256, 256.0
t = torch.arange(n) / fs
sig = rt.Tensor(torch.sin(2 * math.pi * 20 * t) + 0.5 * torch.sin(2 * math.pi * 50.5 * t))
mag = rt.Tensor(sig.rfft().data.abs())
peaks = torch.topk(mag.data, 2).indices.sort().values.tolist()
print("strongest bins (Hz):", peaks, "(tones at 20 and 50.5 Hz)")
leak_plain = float(mag.data[70:].max())
leak_hann = float(sig.apply_window("hann").rfft().data.abs()[70:].max())
print("leakage far from the tones: rectangular %.3f, Hann window %.5f" % (leak_plain, leak_hann))
back = sig.fft().ifft()
print("ifft(fft(x)) == x:", bool(torch.allclose(back.real_part().data, sig.data, atol=1e-5)))
shifted = rt.Tensor(torch.arange(8.0)).fftshift()
print("fftshift:", shifted.as_slice(), " ifftshift restores:", shifted.ifftshift().as_slice() == list(map(float, range(8))))
a, b = torch.randn(64), torch.randn(64)
direct = torch.stack([(a * b.flip(0).roll(k + 1)).sum() for k in range(64)])                    # c[k] = sum_j a[j] b[(k - j) mod n]
via_fft = rt.Tensor(rt.Tensor(a).fft().data * rt.Tensor(b).fft().data).ifft().real_part().data
print("convolution theorem: max difference %.2e" % float((direct - via_fft).abs().max()))
