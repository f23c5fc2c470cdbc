//! `GrindOps` for both Blake2s channels (`core/proof_of_work.rs:3-7`) and the `BackendForChannel` markers
//! (`prover/backend/mod.rs:34-37`).
//!
//! The prefixed digest `H(POW_PREFIX, [0; 12], digest, pow_bits)` is one small host hash, computed exactly as the
//! verifier recomputes it (`core/channel/blake2s.rs:122-140`); the search over nonces runs on the device and returns
//! the smallest `(hi << 32) | lo`, `lo < 2^20`, which is what `simd/grind.rs:18-93` returns. The reference's CUDA
//! backend sends the M31-output channel to the SIMD backend (`cuda/backend.rs:44-48`); here both variants run on the
//! device.
use stwo::core::channel::blake2s::Blake2sChannelGeneric;
use stwo::core::fields::m31::P;
use stwo::core::proof_of_work::GrindOps;
use stwo::core::vcs::blake2_hash::Blake2sHasherGeneric;
use stwo::core::vcs::blake2_merkle::{Blake2sM31MerkleChannel, Blake2sMerkleChannel};
use stwo::prover::backend::BackendForChannel;

use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;

impl<const IS_M31_OUTPUT: bool> GrindOps<Blake2sChannelGeneric<IS_M31_OUTPUT>> for B200Backend {
    fn grind(channel: &Blake2sChannelGeneric<IS_M31_OUTPUT>, pow_bits: u32) -> u64 {
        assert!(pow_bits <= 32, "pow_bits > 32 is not supported");
        let mut hasher = Blake2sHasherGeneric::<IS_M31_OUTPUT>::default();
        hasher.update(&Blake2sChannelGeneric::<IS_M31_OUTPUT>::POW_PREFIX.to_le_bytes());
        hasher.update(&[0_u8; 12]);
        hasher.update(&channel.digest().0[..]);
        hasher.update(&pow_bits.to_le_bytes());
        let prefixed: [u8; 32] = hasher.finalize().0;
        let prefixed_words: [u32; 8] = bytemuck::cast(prefixed);

        let mut nonce = 0u64;
        check(unsafe { ffi::zkb_grind(ctx(), prefixed_words.as_ptr(), pow_bits as i32, IS_M31_OUTPUT as i32, &mut nonce) });
        assert!(((nonce >> 32) as u32) < P && (nonce as u32) < P, "nonce halves are not reduced modulo the M31 prime");
        nonce
    }
}

impl BackendForChannel<Blake2sMerkleChannel> for B200Backend {}
impl BackendForChannel<Blake2sM31MerkleChannel> for B200Backend {}
