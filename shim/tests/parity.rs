//! Parity of `B200Backend` against the reference's own `SimdBackend` and `CpuBackend` on seeded inputs: every trait
//! method is run through both and the results compared word for word. Needs a B200 and `libzkb200.so`
//! (`ZKB200_LIB_DIR`); run with `cargo test --release -- --test-threads 1` (one library context per process).
//!
//! These are the checks the Python suite makes against the C restatement of the same algorithms
//! (`tests/test_gpu_ops.py`, `tests/test_gpu_protocols.py`), made here against the reference's Rust directly.
use rand::rngs::SmallRng;
use rand::{Rng, SeedableRng};
use stwo::core::channel::{Blake2sM31Channel, Channel};
use stwo::core::fields::m31::BaseField;
use stwo::core::fields::qm31::SecureField;
use stwo::core::poly::circle::CanonicCoset;
use stwo::core::proof_of_work::GrindOps;
use stwo::core::vcs::blake2_merkle::Blake2sM31MerkleHasher;
use stwo::prover::backend::simd::SimdBackend;
use stwo::prover::backend::{Col, Column, ColumnOps, CpuBackend};
use stwo::prover::fri::FriOps;
use stwo::prover::line::LineEvaluation;
use stwo::prover::lookups::gkr_prover::{GkrOps, Layer};
use stwo::prover::lookups::mle::Mle;
use stwo::prover::poly::circle::{CircleEvaluation, PolyOps, SecureEvaluation};
use stwo::prover::poly::BitReversedOrder;
use stwo::prover::secure_column::SecureColumnByCoords;
use stwo::prover::vcs::ops::MerkleOps;
use zkb200_backend::{init, B200Backend};

const LOGS: [u32; 4] = [4, 7, 12, 16];

fn base(rng: &mut SmallRng, n: usize) -> Vec<BaseField> { (0..n).map(|_| BaseField::from(rng.gen::<u32>() % ((1 << 31) - 1))).collect() }
fn secure(rng: &mut SmallRng, n: usize) -> Vec<SecureField> {
    (0..n).map(|_| { let b = base(rng, 4); SecureField::from_m31_array([b[0], b[1], b[2], b[3]]) }).collect()
}
fn by_coords<B: ColumnOps<BaseField>>(v: &[SecureField]) -> SecureColumnByCoords<B> {
    SecureColumnByCoords { columns: [0, 1, 2, 3].map(|k| v.iter().map(|q| q.to_m31_array()[k]).collect()) }
}

#[test]
fn columns_bit_reverse_and_gather() {
    init(0, 20);
    let mut rng = SmallRng::seed_from_u64(1);
    for log in LOGS {
        let v = base(&mut rng, 1 << log);
        let mut a: Col<B200Backend, BaseField> = v.iter().copied().collect();
        let mut b: Col<SimdBackend, BaseField> = v.iter().copied().collect();
        <B200Backend as ColumnOps<BaseField>>::bit_reverse_column(&mut a);
        <SimdBackend as ColumnOps<BaseField>>::bit_reverse_column(&mut b);
        assert_eq!(a.to_cpu(), b.to_cpu());
        let idx: Vec<usize> = (0..37).map(|_| rng.gen::<usize>() % (1 << log)).collect();
        assert_eq!(a.batch_at(&idx), b.batch_at(&idx));
        let q = secure(&mut rng, 1 << log);
        let mut a: Col<B200Backend, SecureField> = q.iter().copied().collect();
        let mut b: Col<CpuBackend, SecureField> = q.iter().copied().collect();
        <B200Backend as ColumnOps<SecureField>>::bit_reverse_column(&mut a);
        <CpuBackend as ColumnOps<SecureField>>::bit_reverse_column(&mut b);
        assert_eq!(a.to_cpu(), b.to_cpu());
    }
}

#[test]
fn poly_ops() {
    init(0, 20);
    let mut rng = SmallRng::seed_from_u64(2);
    for log in LOGS {
        let v = base(&mut rng, 1 << log);
        let domain = CanonicCoset::new(log).circle_domain();
        let big = CanonicCoset::new(log + 2).circle_domain();
        let (tw_a, tw_b) = (B200Backend::precompute_twiddles(big.half_coset), SimdBackend::precompute_twiddles(big.half_coset));
        let ea = CircleEvaluation::<B200Backend, BaseField, BitReversedOrder>::new(domain, v.iter().copied().collect());
        let eb = CircleEvaluation::<SimdBackend, BaseField, BitReversedOrder>::new(domain, v.iter().copied().collect());
        let (pa, pb) = (B200Backend::interpolate(ea.clone(), &tw_a), SimdBackend::interpolate(eb.clone(), &tw_b));
        assert_eq!(pa.coeffs.to_cpu(), pb.coeffs.to_cpu());
        assert_eq!(B200Backend::evaluate(&pa, big, &tw_a).values.to_cpu(), SimdBackend::evaluate(&pb, big, &tw_b).values.to_cpu());
        assert_eq!(B200Backend::extend(&pa, log + 1).coeffs.to_cpu(), SimdBackend::extend(&pb, log + 1).coeffs.to_cpu());
        let point = stwo::core::circle::SECURE_FIELD_CIRCLE_GEN.mul(rng.gen::<u64>() as u128);
        let want = SimdBackend::eval_at_point(&pb, point);
        assert_eq!(B200Backend::eval_at_point(&pa, point), want);
        let (wa, wb) = (B200Backend::barycentric_weights(CanonicCoset::new(log), point), SimdBackend::barycentric_weights(CanonicCoset::new(log), point));
        assert_eq!(wa.to_cpu(), wb.to_cpu());
        assert_eq!(B200Backend::barycentric_eval_at_point(&ea, &wa), want);
        assert_eq!(B200Backend::eval_at_point_by_folding(&ea, point, &tw_a), want);
    }
}

#[test]
fn merkle_layers() {
    init(0, 20);
    let mut rng = SmallRng::seed_from_u64(3);
    for log in [4u32, 9, 14] {
        let cols: Vec<Vec<BaseField>> = (0..5).map(|_| base(&mut rng, 1 << log)).collect();
        let ca: Vec<Col<B200Backend, BaseField>> = cols.iter().map(|c| c.iter().copied().collect()).collect();
        let cb: Vec<Col<SimdBackend, BaseField>> = cols.iter().map(|c| c.iter().copied().collect()).collect();
        let la = <B200Backend as MerkleOps<Blake2sM31MerkleHasher>>::commit_on_layer(log, None, &ca.iter().collect::<Vec<_>>());
        let lb = <SimdBackend as MerkleOps<Blake2sM31MerkleHasher>>::commit_on_layer(log, None, &cb.iter().collect::<Vec<_>>());
        assert_eq!(la.to_cpu(), lb.to_cpu());
        let ua = <B200Backend as MerkleOps<Blake2sM31MerkleHasher>>::commit_on_layer(log - 1, Some(&la), &[]);
        let ub = <SimdBackend as MerkleOps<Blake2sM31MerkleHasher>>::commit_on_layer(log - 1, Some(&lb), &[]);
        assert_eq!(ua.to_cpu(), ub.to_cpu());
    }
}

#[test]
fn fri_folds() {
    init(0, 20);
    let mut rng = SmallRng::seed_from_u64(4);
    for log in [5u32, 10, 15] {
        let v = secure(&mut rng, 1 << log);
        let alpha = secure(&mut rng, 1)[0];
        let domain = CanonicCoset::new(log).circle_domain();
        let (tw_a, tw_b) = (B200Backend::precompute_twiddles(domain.half_coset), CpuBackend::precompute_twiddles(domain.half_coset));
        let sa = SecureEvaluation::<B200Backend, BitReversedOrder>::new(domain, by_coords(&v));
        let sb = SecureEvaluation::<CpuBackend, BitReversedOrder>::new(domain, by_coords(&v));
        let line = stwo::core::poly::line::LineDomain::new(domain.half_coset);
        let mut da = LineEvaluation::<B200Backend>::new_zero(line);
        let mut db = LineEvaluation::<CpuBackend>::new_zero(line);
        B200Backend::fold_circle_into_line(&mut da, &sa, alpha, &tw_a);
        CpuBackend::fold_circle_into_line(&mut db, &sb, alpha, &tw_b);
        assert_eq!(da.values.to_vec(), db.values.to_vec());
        for step in [1u32, 2, 3] {
            let fa = B200Backend::fold_line(&da, alpha, &tw_a, step);
            let fb = CpuBackend::fold_line(&db, alpha, &tw_b, step);
            assert_eq!(fa.values.to_vec(), fb.values.to_vec());
        }
    }
}

#[test]
fn gkr_layers_and_round_polynomials() {
    init(0, 20);
    let mut rng = SmallRng::seed_from_u64(5);
    for log in [3usize, 8, 13] {
        let (num, den, mult) = (secure(&mut rng, 1 << log), secure(&mut rng, 1 << log), base(&mut rng, 1 << log));
        let layers_a: Vec<Layer<B200Backend>> = vec![
            Layer::GrandProduct(Mle::new(den.iter().copied().collect())),
            Layer::LogUpGeneric { numerators: Mle::new(num.iter().copied().collect()), denominators: Mle::new(den.iter().copied().collect()) },
            Layer::LogUpMultiplicities { numerators: Mle::new(mult.iter().copied().collect()), denominators: Mle::new(den.iter().copied().collect()) },
            Layer::LogUpSingles { denominators: Mle::new(den.iter().copied().collect()) },
        ];
        let layers_b: Vec<Layer<CpuBackend>> = vec![
            Layer::GrandProduct(Mle::new(den.clone())),
            Layer::LogUpGeneric { numerators: Mle::new(num.clone()), denominators: Mle::new(den.clone()) },
            Layer::LogUpMultiplicities { numerators: Mle::new(mult.clone()), denominators: Mle::new(den.clone()) },
            Layer::LogUpSingles { denominators: Mle::new(den.clone()) },
        ];
        let y = secure(&mut rng, log - 1);
        let v = secure(&mut rng, 1)[0];
        assert_eq!(B200Backend::gen_eq_evals(&y, v).to_cpu(), CpuBackend::gen_eq_evals(&y, v).to_cpu());
        for (la, lb) in layers_a.iter().zip(&layers_b) {
            assert_eq!(B200Backend::next_layer(la).to_cpu_layer_words(), CpuBackend::next_layer(lb).to_cpu_layer_words());
        }
        // One whole GKR proof per layer kind through the generic prover: every round polynomial, every
        // fix_first_variable and every mask goes into the transcript, so equal proofs mean equal operators.
        for (la, lb) in layers_a.into_iter().zip(layers_b) {
            let (pa, _) = stwo::prover::lookups::gkr_prover::prove_batch(&mut Blake2sM31Channel::default(), vec![la]);
            let (pb, _) = stwo::prover::lookups::gkr_prover::prove_batch(&mut Blake2sM31Channel::default(), vec![lb]);
            assert_eq!(format!("{pa:?}"), format!("{pb:?}"));
        }
    }
}

/// The words of a layer's columns, in declaration order (test helper; the reference's `Layer::to_cpu` is private).
trait LayerWords { fn to_cpu_layer_words(&self) -> Vec<Vec<SecureField>>; }
impl<B: GkrOps> LayerWords for Layer<B> {
    fn to_cpu_layer_words(&self) -> Vec<Vec<SecureField>> {
        match self {
            Layer::GrandProduct(c) => vec![c.to_cpu()],
            Layer::LogUpGeneric { numerators, denominators } => vec![numerators.to_cpu(), denominators.to_cpu()],
            Layer::LogUpMultiplicities { numerators, denominators } => {
                vec![numerators.to_cpu().into_iter().map(SecureField::from).collect(), denominators.to_cpu()]
            }
            Layer::LogUpSingles { denominators } => vec![denominators.to_cpu()],
        }
    }
}

#[test]
fn grind_finds_the_same_nonce() {
    init(0, 20);
    for (seed, bits) in [(7u32, 8u32), (8, 16), (9, 20)] {
        let mut channel = Blake2sM31Channel::default();
        channel.mix_u64(seed as u64);
        assert_eq!(<B200Backend as GrindOps<_>>::grind(&channel, bits), <SimdBackend as GrindOps<_>>::grind(&channel, bits));
    }
}
