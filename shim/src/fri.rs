//! `FriOps` (`prover/fri.rs:48-86`).
use stwo::core::fields::qm31::SecureField;
use stwo::prover::backend::Column;
use stwo::prover::fri::FriOps;
use stwo::prover::line::LineEvaluation;
use stwo::prover::poly::circle::SecureEvaluation;
use stwo::prover::poly::twiddles::TwiddleTree;
use stwo::prover::poly::BitReversedOrder;
use stwo::prover::secure_column::SecureColumnByCoords;

use crate::column::{B200BaseColumn, DeviceWords};
use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;

pub(crate) fn coords(c: &SecureColumnByCoords<B200Backend>) -> [*const u32; 4] { [0, 1, 2, 3].map(|k| c.columns[k].0.ptr as *const u32) }
pub(crate) fn coords_mut(c: &mut SecureColumnByCoords<B200Backend>) -> [*mut u32; 4] { [0, 1, 2, 3].map(|k| c.columns[k].0.ptr) }
pub(crate) fn new_secure(len: usize) -> SecureColumnByCoords<B200Backend> {
    SecureColumnByCoords { columns: [0, 1, 2, 3].map(|_| B200BaseColumn(DeviceWords::uninit(len))) }
}
pub(crate) fn words(q: SecureField) -> [u32; 4] { q.to_m31_array().map(|m| m.0) }

impl FriOps for B200Backend {
    fn fold_line(eval: &LineEvaluation<Self>, alpha: SecureField, _twiddles: &TwiddleTree<Self>, fold_step: u32) -> LineEvaluation<Self> {
        assert!(eval.len() >= 2 && fold_step >= 1);
        // cpu/fri.rs:15-30: `fold_step` folds, the challenge squared between them
        let mut domain = eval.domain();
        let mut cur: Option<SecureColumnByCoords<Self>> = None;
        let mut a = alpha;
        for _ in 0..fold_step {
            let src = cur.as_ref().unwrap_or(&eval.values);
            let n = src.len();
            let mut out = new_secure(n / 2);
            check(unsafe { ffi::zkb_fold_line(ctx(), coords_mut(&mut out).as_ptr(), coords(src).as_ptr(), n.ilog2() as i32, words(a).as_ptr()) });
            cur = Some(out);
            domain = domain.double();
            a = a * a;
        }
        LineEvaluation::new(domain, cur.unwrap())
    }

    fn fold_circle_into_line(dst: &mut LineEvaluation<Self>, src: &SecureEvaluation<Self, BitReversedOrder>, alpha: SecureField, _twiddles: &TwiddleTree<Self>) {
        assert_eq!(src.len() >> 1, dst.len());
        let log = src.domain.log_size();
        check(unsafe { ffi::zkb_fold_circle_into_line(ctx(), coords_mut(&mut dst.values).as_ptr(), coords(&src.values).as_ptr(), log as i32, words(alpha).as_ptr()) });
    }

    fn decompose(_eval: &SecureEvaluation<Self, BitReversedOrder>) -> (SecureEvaluation<Self, BitReversedOrder>, SecureField) {
        // Not used by the prover and `todo!()` in the reference's own device backend (backend/cuda/fri.rs:71-77);
        // zkb_fri_decompose returns ZKB_EINVAL with the same explanation.
        unimplemented!("FriOps::decompose: every polynomial that enters FRI already lies in the FFT space")
    }
}
