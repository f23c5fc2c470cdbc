//! `MerkleOps::commit_on_layer` for both Blake2s hashers (`prover/vcs/ops.rs:24-29`).
use stwo::core::fields::m31::BaseField;
use stwo::core::vcs::blake2_hash::Blake2sHash;
use stwo::core::vcs::blake2_merkle::{Blake2sM31MerkleHasher, Blake2sMerkleHasher};
use stwo::prover::backend::Col;
use stwo::prover::vcs::ops::MerkleOps;

use crate::column::{B200HashColumn, DeviceWords};
use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;

fn commit(log_size: u32, prev: Option<&B200HashColumn>, columns: &[&Col<B200Backend, BaseField>], m31: bool) -> B200HashColumn {
    let out = DeviceWords::uninit(8usize << log_size);
    let ptrs: Vec<*const u32> = columns.iter().map(|c| c.0.ptr as *const u32).collect();
    let prev_ptr = prev.map_or(std::ptr::null(), |p| p.0.ptr as *const u32);
    check(unsafe { ffi::zkb_merkle_layer(ctx(), log_size as i32, prev_ptr, ptrs.as_ptr(), ptrs.len() as i32, m31 as i32, out.ptr) });
    B200HashColumn(out)
}

impl MerkleOps<Blake2sM31MerkleHasher> for B200Backend {
    fn commit_on_layer(log_size: u32, prev_layer: Option<&Col<Self, Blake2sHash>>, columns: &[&Col<Self, BaseField>]) -> Col<Self, Blake2sHash> {
        commit(log_size, prev_layer, columns, true)
    }
}
impl MerkleOps<Blake2sMerkleHasher> for B200Backend {
    fn commit_on_layer(log_size: u32, prev_layer: Option<&Col<Self, Blake2sHash>>, columns: &[&Col<Self, BaseField>]) -> Col<Self, Blake2sHash> {
        commit(log_size, prev_layer, columns, false)
    }
}
