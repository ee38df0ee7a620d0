"""The networks of the benchmark configurations, assembled from the layer mirrors (layers.py) the way the reference's
models assemble its layer classes (cuda/netmodel/cmodel_basicgan.cu.h:CreateGenerator/CreateDiscriminator build the same
chains from CNetLayerLinear, CNetLayerBackConvolution / CNetLayerConvolution, CNetLayerBatchNormalization and
CNetLayerFunction)."""
import torch

from . import ops
from .lib import load
from .layers import (AdamCorrections, Net, NetLayerBackConvolution, NetLayerBatchNormalization, NetLayerBatchNormalizationFunction,
                     NetLayerConvolution, NetLayerFunction, NetLayerLinear, NetLayerMaxPooling, NetLayerUpSampling)


def _bn_function(spec, fused, leaky_slope):
    """Batch normalisation followed by LeakyReLU: two layers as in the reference, or the fused pair.  The fused pair saves
    two passes over the activations, which pays on tensors beyond L2; at the DCGAN sizes (a few MB, resident in L2) the
    extra phase inside the latency-bound normalisation kernels costs more than two tiny launches (measured: 1.26 ms against
    1.24 ms per step), so the nets default to the two layers."""
    if fused:
        spec.append((NetLayerBatchNormalizationFunction, dict(func="leaky_relu", leaky_slope=leaky_slope)))
    else:
        spec.append((NetLayerBatchNormalization, {}))
        spec.append((NetLayerFunction, dict(func="leaky_relu", leaky_slope=leaky_slope)))


def dcgan_generator(batch, noise=100, base=512, widths=(256, 128, 64, 3), leaky_slope=0.2, seed=2, fused=False, peer=False, channel=0):
    """z[noise] -> Linear to base x 4 x 4 -> 4x4 stride-2 transposed convolutions to widths[-1] x 64 x 64; batch
    normalisation and LeakyReLU after every stage but the last, tanh at the output."""
    spec = [(NetLayerLinear, dict(neurons=base * 16)), ("reshape", (base, 4, 4))]
    for i, width in enumerate(widths):
        spec.append((NetLayerBackConvolution, dict(kernel_amount=width, kernel_size=4, stride=2, padding=1)))
        if i + 1 < len(widths):
            _bn_function(spec, fused, leaky_slope)
    spec.append((NetLayerFunction, dict(func="tanh")))
    return Net((1, noise, 1), batch, spec, seed=seed, peer=peer, channel=channel)


def dcgan_discriminator(batch, image=(3, 64, 64), widths=(64, 128, 256, 512), leaky_slope=0.2, seed=3, fused=False, peer=False, channel=0):
    """image -> 4x4 stride-2 convolutions with batch normalisation and LeakyReLU -> Linear to one logit -> sigmoid."""
    spec = []
    for width in widths:
        spec.append((NetLayerConvolution, dict(kernel_amount=width, kernel_size=4, stride=2, padding=1)))
        _bn_function(spec, fused, leaky_slope)
    spec.append((NetLayerLinear, dict(neurons=1)))
    spec.append((NetLayerFunction, dict(func="sigmoid")))
    return Net(image, batch, spec, seed=seed, peer=peer, channel=channel)


class DCGANStep:
    """One combined training step of the two networks on a rank's shard of the mini-batch: generator forward, discriminator
    forward on the generated images, the discriminator's backward pass with its weight gradients and the error at its
    input, the generator's backward pass with its weight gradients, one all-reduce per gradient arena and one Adam
    launch per net.  The error at the discriminator's output is output - label (the gradient of binary cross-entropy with
    respect to the logit, formed as in cuda/netmodel/cmodel_basicgan.cu.h:352-376 but on the device)."""

    def __init__(self, batch, world=1, widths_g=(256, 128, 64, 3), widths_d=(64, 128, 256, 512), base=512, noise=100, leaky_slope=0.2,
                 use_graph=True, fused=False, update="fused", overlap=False, lean=True):
        """update (several ranks): "fused" -- the library's reduce-scatter + Adam + all-gather kernel over NVLink peer memory,
        one launch per net on the main stream; "nccl" -- an NCCL all-reduce of each gradient arena on a side stream followed
        by the Adam launch.  overlap: the discriminator's exchange on a side stream beside the generator's backward pass
        (measured on 2 GPUs: no gain -- the exchange kernel's CTAs take whole SMs from the backward pass for as long as they
        run -- so it is off by default)."""
        self.batch, self.world, self.overlap = batch, world, overlap
        self.update = update if world > 1 else "local"
        peer = self.update == "fused"
        if peer:
            from .dp import PeerBuffer
            peer = PeerBuffer(32 << 20)         # one buffer for both nets (weights + gradients of ~6.4 M parameters, with room to spare)
        self.G = dcgan_generator(batch, noise, base, widths_g, leaky_slope, fused=fused, peer=peer, channel=1)
        self.D = dcgan_discriminator(batch, self.G.out_shape, widths_d, leaky_slope, fused=fused, peer=peer, channel=0)
        if lean:    # function layers folded into the convolution behind them do not write an output tensor nobody reads
            self.G.fold_functions(True, materialise=False)
            self.D.fold_functions(True, materialise=False)
        self.G.broadcast_weights()
        self.D.broadcast_weights()
        self.error = torch.empty((batch, 1, 1, 1), device="cuda")
        self.z = torch.empty((batch, 1, noise, 1), device="cuda")
        self.labels = torch.empty((batch, 1, 1, 1), device="cuda")
        self.iteration = 0
        self.use_graph, self.graph, self.eager_steps = use_graph, None, 0
        self.out = None
        self.side_d = torch.cuda.Stream() if (self.update == "nccl" or (self.update == "fused" and overlap)) else None
        self.side_g = torch.cuda.Stream() if self.update == "nccl" else None
        self.corr = AdamCorrections()

    def _step(self, speed):
        """The whole step with fixed launch arguments (capturable): gradients, all-reduces, Adam.  With several ranks the
        discriminator's gradient arena is all-reduced on a side stream while the generator's backward pass runs, and the
        generator's while the discriminator's Adam update runs."""
        main = torch.cuda.current_stream()
        self.G.TrainingResetDeltaWeight()
        self.D.TrainingResetDeltaWeight()
        Net.PrepackWeights([self.G, self.D])        # the weights of both nets change only at the end of the step
        fake = self.G.Forward(self.z)
        out = self.D.Forward(fake)
        ops.CTensorMath.Sub(self.error, out, self.labels)
        d_image = self.D.TrainingBackward(self.error, True, need_input_error=True)
        if self.update == "fused":
            # the generator's backward pass reads the error at the discriminator's input, not the discriminator's weights
            # and the two nets use different channels of their communicators, so the discriminator's exchange may run beside it
            if self.overlap:
                self.side_d.wait_stream(main)
                with torch.cuda.stream(self.side_d):
                    self.D.TrainingUpdateWeightFused(speed, None, batch_scale=self.world, corrections=self.corr.device)
                self.G.TrainingBackward(d_image, True)
                self.G.TrainingUpdateWeightFused(speed, None, batch_scale=self.world, corrections=self.corr.device)
                main.wait_stream(self.side_d)
                return out
            # default: both nets in one exchange launch after the generator's backward pass (one pair of device-side barriers
            # per step instead of two)
            self.G.TrainingBackward(d_image, True)
            Net.TrainingUpdateWeightFusedTogether([self.D, self.G], speed, None, batch_scale=self.world, corrections=self.corr.device)
            return out
        if self.world > 1:
            self.side_d.wait_stream(main)
            with torch.cuda.stream(self.side_d):
                self.D.grads.all_reduce()
        self.G.TrainingBackward(d_image, True)
        if self.world > 1:
            self.side_g.wait_stream(main)
            with torch.cuda.stream(self.side_g):
                self.G.grads.all_reduce()
            main.wait_stream(self.side_d)
        self.D.TrainingUpdateWeight(speed, None, batch_scale=self.world, corrections=self.corr.device)
        if self.world > 1:
            main.wait_stream(self.side_g)
        self.G.TrainingUpdateWeight(speed, None, batch_scale=self.world, corrections=self.corr.device)
        return out

    def __call__(self, z, labels, speed=2e-4):
        """The step is a chain of over a hundred launches of a few microseconds each, so after two eager steps (which size
        every scratch buffer of the library) it is captured once in a CUDA graph and replayed.  Adam's bias corrections for
        the step are refreshed in device memory before each replay (layers.AdamCorrections), so the two Adam launches are
        part of the graph.  While a replay is in flight no other call into the library may run on the same device: the
        Linear layers' products inside the graph use the device's shared scratch arena."""
        self.iteration += 1
        if z.data_ptr() != self.z.data_ptr():
            self.z.copy_(z, non_blocking=True)
        if labels.data_ptr() != self.labels.data_ptr():
            self.labels.copy_(labels, non_blocking=True)
        self.corr.set(self.iteration)
        if self.graph is not None and (load().b200_scratch_bytes() != self.scratch_bytes or speed != self.graph_speed or
                                       load().b200_get_precision() != self.graph_precision):
            # stale addresses (the library's scratch arena moved), another learning rate, or another precision mode than the
            # one the captured launches were chosen in
            self.graph, self.eager_steps = None, 0
        if self.use_graph and self.graph is None and self.eager_steps >= 2:
            ops.stream_status()
            self.scratch_bytes, self.graph_speed, self.graph_precision = load().b200_scratch_bytes(), speed, load().b200_get_precision()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self.out = self._step(speed)
            self.graph = graph
        if self.graph is not None:
            self.graph.replay()
        else:
            self.out = self._step(speed)
            self.eager_steps += 1
        return self.out



def vae_encoder(batch, image=(3, 128, 128), widths=(32, 64, 128, 256), leaky_slope=0.1, seed=4):
    """image -> 4 x (3x3 convolution, LeakyReLU, 2x2 max-pooling)."""
    spec = []
    for width in widths:
        spec.append((NetLayerConvolution, dict(kernel_amount=width, kernel_size=3, stride=1, padding=1)))
        spec.append((NetLayerFunction, dict(func="leaky_relu", leaky_slope=leaky_slope)))
        spec.append((NetLayerMaxPooling, dict(pooling=2)))
    return Net(image, batch, spec, seed=seed)


def vae_decoder(batch, latent=256, start=(256, 8, 8), widths=(128, 64, 32, 3), leaky_slope=0.1, seed=5):
    """latent -> Linear to start -> 4 x (2x upsampling, 3x3 convolution), LeakyReLU between, sigmoid at the output."""
    spec = [(NetLayerLinear, dict(neurons=start[0] * start[1] * start[2])), ("reshape", tuple(start)),
            (NetLayerFunction, dict(func="leaky_relu", leaky_slope=leaky_slope))]
    for i, width in enumerate(widths):
        spec.append((NetLayerUpSampling, dict(factor=2)))
        spec.append((NetLayerConvolution, dict(kernel_amount=width, kernel_size=3, stride=1, padding=1)))
        spec.append((NetLayerFunction, dict(func="leaky_relu", leaky_slope=leaky_slope) if i + 1 < len(widths) else dict(func="sigmoid")))
    return Net((1, latent, 1), batch, spec, seed=seed)


class VAEStep:
    """One training step of the convolutional VAE on a rank's shard: encoder, the two Linear heads (mean and log-variance),
    the reparameterised latent with caller-supplied noise (netlayer/cnetlayervaecoderoutput.cu.h:244-287), decoder; error
    2(x_hat - x)/numel at the output plus the Kullback-Leibler terms at the heads (:424-460); backward through all four
    nets with weight gradients, one all-reduce per gradient arena, Adam on every net."""

    def __init__(self, batch, world=1, image=(3, 128, 128), widths=(32, 64, 128, 256), latent=256, kl_speed=1.0, leaky_slope=0.1):
        self.batch, self.world, self.kl_speed = batch, world, kl_speed
        self.encoder = vae_encoder(batch, image, widths, leaky_slope)
        feat = self.encoder.out_shape
        self.mu = Net(feat, batch, [(NetLayerLinear, dict(neurons=latent))], seed=6)
        self.logvar = Net(feat, batch, [(NetLayerLinear, dict(neurons=latent))], seed=7)
        self.decoder = vae_decoder(batch, latent, feat, tuple(widths[-2::-1]) + (image[0],), leaky_slope)
        assert self.decoder.out_shape == tuple(image), (self.decoder.out_shape, image)
        self.nets = (self.encoder, self.mu, self.logvar, self.decoder)
        for net in self.nets:
            net.broadcast_weights()
        self.error = torch.empty((batch,) + tuple(image), device="cuda")
        self.feat_error = torch.empty((batch,) + feat, device="cuda")
        self.iteration = 0
        self.kl = None

    def __call__(self, x, eps, speed=1e-3, want_kl=False):
        self.iteration += 1
        for net in self.nets:
            net.TrainingResetDeltaWeight()
        Net.PrepackWeights(self.nets)               # all weights change only at the end of the step
        feat = self.encoder.Forward(x)
        mu, logvar = self.mu.Forward(feat), self.logvar.Forward(feat)
        z, self.kl = ops.vae_forward(mu, logvar, eps.view(mu.shape), want_kl=want_kl)
        x_hat = self.decoder.Forward(z)
        ops.CTensorMath.Sub(self.error, x_hat, x, 2.0 / x[0].numel(), 2.0 / x[0].numel())
        d_z = self.decoder.TrainingBackward(self.error, True, need_input_error=True)
        d_mu, d_logvar = ops.vae_backward(d_z.view(mu.shape), mu, logvar, eps.view(mu.shape), self.kl_speed)
        e_mu = self.mu.TrainingBackward(d_mu, True, need_input_error=True)
        e_lv = self.logvar.TrainingBackward(d_logvar, True, need_input_error=True)
        ops.CTensorMath.Add(self.feat_error, e_mu, e_lv)
        self.encoder.TrainingBackward(self.feat_error, True)
        for net in self.nets:
            net.grads.all_reduce()
            net.TrainingUpdateWeight(speed, self.iteration, batch_scale=self.world)
        return x_hat


class GANSeparableTrainer:
    """One iteration of the reference's separable GAN training (cuda/netmodel/cmodel_basicgan.cu.h:TrainingSeparable, :700-823)
    on a rank's shard: (1) the discriminator on generated images (TrainingDiscriminatorFake, :327-394), weights updated;
    (2) the discriminator on real images (TrainingDiscriminatorReal, :396-464), weights updated; (3) the generator through
    the discriminator, whose weight gradients are not formed (TrainingGenerator, :466-539), generator weights updated.
    The errors at the discriminator's output are the reference's hinge rules -- 1 where D(fake) > -1, -1 where D(real) < 1,
    -1 for the generator pass -- formed on the device instead of by a per-sample host loop over a read-back tensor."""

    def __init__(self, generator, discriminator, world=1):
        self.G, self.D, self.world = generator, discriminator, world
        self.batch = generator.batch
        self.error = torch.empty((self.batch, 1, 1, 1), device="cuda")
        self.minus_one = torch.full((self.batch, 1, 1, 1), -1.0, device="cuda")
        self.G.broadcast_weights()
        self.D.broadcast_weights()

    def _hinge(self, out, real):
        """fake pass: 1 where out > -1 else 0; real pass: -1 where out < 1 else 0."""
        out = out.view(self.batch, 1, 1, 1)
        ops.CTensorMath.Set(self.error, out, -1.0 if real else 1.0, 1.0)      # 1 - out  /  out + 1
        ops.CTensorMath.Signum(self.error)
        ops.CTensorMath.Clip(self.error, 0.0, 1.0)
        if real:
            ops.CTensorMath.Set(self.error, self.error, -1.0, 0.0)
        return self.error

    def _update(self, net, speed, iteration):
        net.grads.all_reduce()
        net.TrainingUpdateWeight(speed, iteration, batch_scale=self.world)

    def TrainingSeparable(self, noise_for_discriminator, real_images, noise_for_generator, disc_speed, gen_speed, iteration):
        G, D = self.G, self.D
        D.TrainingResetDeltaWeight()
        D.TrainingBackward(self._hinge(D.Forward(G.Forward(noise_for_discriminator)), real=False), True)
        self._update(D, disc_speed, iteration)
        D.TrainingResetDeltaWeight()
        D.TrainingBackward(self._hinge(D.Forward(real_images), real=True), True)
        self._update(D, disc_speed, iteration)
        G.TrainingResetDeltaWeight()
        answers = D.Forward(G.Forward(noise_for_generator))
        d_image = D.TrainingBackward(self.minus_one, False, need_input_error=True)
        G.TrainingBackward(d_image, True)
        self._update(G, gen_speed, iteration)
        return answers
